// seq_recurrent.cu -- the parts of the token-major models that carry per-sequence STATE instead of cache pages, all in
// float32: a short causal convolution over time in front of a sublayer, and linear attention with a fixed decay per head.
//
//   causal_conv_rows   u_t = h_t + sum_j w[:, j] h_(t - taps + 1 + j), channel by channel.  Inputs of the same step come
//                      from the rows before it (rows of a sequence are consecutive), older ones from the sequence's state:
//                      a ring of taps - 1 rows per slot, position p at ring row p mod (taps - 1); positions below 0 are zero.
//   causal_conv_state  the step's last taps - 1 inputs of every sequence enter the ring (a launch of its own: rows of the
//                      same launch still read the old ring).  With the ring kept twice per slot (read one copy, write the
//                      other, the step's parity says which) the rows' launch updates it itself.
//   linear_prep        per token and head on the fused projection row: activation of q / k / v, rotation of q and k (the
//                      first rot_dims elements, element i paired with i + rot_dims / 2), k scaled.
//   linear_attention   S_t = a_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  A block owns one (sequence, head, slice of value
//                      columns): it keeps S [D][slice] in shared memory, walks the step's tokens in chunks of 32 --
//                      scores q_t.k_s a^(t-s) inside the chunk, the carried state for everything before it -- and leaves
//                      the state in the slot's array.  A sequence whose first position is 0 starts from zero, whatever the
//                      slot held.  One decoded token is a chunk of one.
//   linear_finish      the heads' outputs divided by their root mean square (over all heads with a weight, or head by head
//                      without one), times sigmoid or silu of the gate columns, times a constant.
#include "common.cuh"
#include "../../include/pgk_b200.h"

using namespace pgk;

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// ---------------------------------------------------------------- causal convolution
struct ConvArgs {
    const float* h; float* u; const float* w; float* state;
    const int* slot; const int* pos; const int* parity; int T, W, taps;
    int ldh, ldu;                        // row strides of h and u (W when the rows are dense)
    int residual, act;                   // residual 1: u = h + conv(h), 0: u = conv(h); act 1: silu on the result
};

// parity == NULL: one ring per slot, updated by causal_conv_state_kernel afterwards.  Otherwise the ring is kept twice per
// slot, [2][taps - 1][W]: the step reads the copy parity[t] of its sequence and this launch writes the other one -- every row
// among the last taps - 1 of its sequence its own input, the sequence's last row also the entries that stay valid when the
// step brought fewer than taps - 1 rows -- so that no block reads what another block of the same launch writes.
__global__ void __launch_bounds__(256) causal_conv_rows_kernel(ConvArgs a) {
    const int t = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
    if (c >= a.W) return;
    const int p = a.pos[t], s = a.slot[t], ring = a.taps - 1, W = a.W;
    const bool twice = a.parity != nullptr;
    const int par = twice ? (a.parity[t] & 1) : 0;
    const float* rin = a.state + ((size_t)s * (twice ? 2 : 1) + par) * ring * W;
    float* rout = a.state + ((size_t)s * 2 + (par ^ 1)) * ring * W;
    const bool last_row = twice && (t + 1 >= a.T || a.slot[t + 1] != s);
    const bool tail_row = twice && ring > 0 && (t + ring >= a.T || a.slot[t + ring] != s);
    const float* w = a.w + (size_t)c * a.taps;
    const float hv = a.h[(size_t)t * a.ldh + c];
    float acc = fmaf(w[a.taps - 1], hv, a.residual ? hv : 0.f);
    for (int k = 1; k < a.taps && k <= p; ++k) {
        const bool instep = t - k >= 0 && a.slot[t - k] == s;
        const float v = instep ? a.h[(size_t)(t - k) * a.ldh + c] : rin[(size_t)((p - k) % ring) * W + c];
        acc = fmaf(w[a.taps - 1 - k], v, acc);
        if (last_row && k < ring && !instep) rout[(size_t)((p - k) % ring) * W + c] = v;
    }
    a.u[(size_t)t * a.ldu + c] = a.act ? silu_f(acc) : acc;
    if (tail_row) rout[(size_t)(p % ring) * W + c] = hv;
}

// seqs [n][4] = (first row, rows, slot, first position); block x = sequence * ring + i: the i-th last row of the sequence
__global__ void __launch_bounds__(256) causal_conv_state_kernel(const float* h, float* state, const int4* seqs, int W, int ring) {
    const int4 sq = seqs[blockIdx.x / ring];
    const int i = blockIdx.x % ring, c = blockIdx.y * 256 + threadIdx.x;
    if (i >= sq.y || c >= W) return;
    const int r = sq.y - 1 - i, p = sq.w + r;
    state[((size_t)sq.z * ring + p % ring) * W + c] = h[(size_t)(sq.x + r) * W + c];
}

// ---------------------------------------------------------------- linear attention: preparation of q / k / v
struct LinPrepArgs {
    float* proj; int ld, H, D, Dv, q_off, k_off, v_off, act, rot_dims;
    const double* inv_freq; float k_scale; const int* pos;
};

// units per token: H query heads, H key heads, H value heads; a warp each
__global__ void __launch_bounds__(128) linear_prep_kernel(LinPrepArgs a) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, u = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (u >= 3 * a.H) return;
    float* row = a.proj + (size_t)t * a.ld;
    if (u >= 2 * a.H) {
        if (!a.act) return;
        float* v = row + a.v_off + (size_t)(u - 2 * a.H) * a.Dv;
        for (int d = lane; d < a.Dv; d += 32) v[d] = silu_f(v[d]);
        return;
    }
    const bool is_k = u >= a.H;
    float* x = row + (is_k ? a.k_off + (size_t)(u - a.H) * a.D : a.q_off + (size_t)u * a.D);
    const float sc = is_k ? a.k_scale : 1.f;
    const int half = a.rot_dims / 2, pos = a.pos[t];
    for (int i = lane; i < half; i += 32) {
        float p0 = x[i], p1 = x[i + half];
        if (a.act) { p0 = silu_f(p0); p1 = silu_f(p1); }
        float sn, cs;
        rope_angle_sincos(pos, a.inv_freq[i], sn, cs);
        x[i] = (p0 * cs - p1 * sn) * sc;
        x[i + half] = (p1 * cs + p0 * sn) * sc;
    }
    for (int d = 2 * half + lane; d < a.D; d += 32) x[d] = (a.act ? silu_f(x[d]) : x[d]) * sc;
}

// ---------------------------------------------------------------- linear attention: the recurrence
constexpr int LC = 32;                  // tokens per chunk

struct LinArgs {
    const float* proj; int ld, q_off, k_off, v_off;
    float* out; int ldo;
    float* state;                        // [slots][H][D][Dv]
    const float* decay;                  // [H]
    const int4* seqs;                    // (first row, rows, slot, first position)
    int H, D, Dv, DS;                    // DS: value columns per block
};

__global__ void __launch_bounds__(256) linear_attention_kernel(LinArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int D = a.D, DS = a.DS, DP = D + 1;
    float* S = sm;                      // [D][DS]
    float* Q = S + D * DS;              // [LC][D + 1]
    float* K = Q + LC * DP;             // [LC][D + 1]
    float* V = K + LC * DP;             // [LC][DS]
    float* A = V + LC * DS;             // [LC][LC + 1]
    float* pw = A + LC * (LC + 1);      // [LC + 1]: decay^i
    const int4 sq = a.seqs[blockIdx.x];
    const int row0 = sq.x, n = sq.y, slot = sq.z, pos0 = sq.w;
    const int h = blockIdx.y, dv0 = blockIdx.z * DS, nd = min(DS, a.Dv - dv0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float dec = a.decay[h];
    float* Sg = a.state + (((size_t)slot * a.H + h) * D) * a.Dv + dv0;
    for (int i = tid; i < D * DS; i += 256) {
        const int d = i / DS, c = i - d * DS;
        S[i] = (pos0 > 0 && c < nd) ? Sg[(size_t)d * a.Dv + c] : 0.f;
    }
    if (tid <= LC) pw[tid] = powf(dec, (float)tid);
    for (int c0 = 0; c0 < n; c0 += LC) {
        const int nc = min(LC, n - c0);
        __syncthreads();
        for (int i = tid; i < nc * D; i += 256) {
            const int r = i / D, d = i - r * D;
            const float* src = a.proj + (size_t)(row0 + c0 + r) * a.ld + (size_t)h * D + d;
            Q[r * DP + d] = src[a.q_off];
            K[r * DP + d] = src[a.k_off];
        }
        for (int i = tid; i < nc * DS; i += 256) {
            const int r = i / DS, c = i - r * DS;
            V[i] = c < nd ? a.proj[(size_t)(row0 + c0 + r) * a.ld + a.v_off + (size_t)h * a.Dv + dv0 + c] : 0.f;
        }
        __syncthreads();
        // scores inside the chunk: lane = key s, the warp's rows t = warp, warp + 8, ...
        for (int t = warp; t < nc; t += 8) {
            float s = 0.f;
            if (lane <= t) {
                const float* q = Q + t * DP;
                const float* k = K + lane * DP;
                for (int d = 0; d < D; ++d) s = fmaf(q[d], k[d], s);
                s *= pw[t - lane];
            }
            A[t * (LC + 1) + lane] = s;
        }
        __syncthreads();
        // outputs: o_t = a^(t + 1) S^T q_t + sum_{s <= t} A[t][s] v_s
        for (int i = tid; i < nc * DS; i += 256) {
            const int t = i / DS, c = i - t * DS;
            if (c >= nd) continue;
            const float* q = Q + t * DP;
            float o = 0.f;
            for (int d = 0; d < D; ++d) o = fmaf(q[d], S[d * DS + c], o);
            o *= pw[t + 1];
            const float* ar = A + t * (LC + 1);
            for (int s = 0; s <= t; ++s) o = fmaf(ar[s], V[s * DS + c], o);
            a.out[(size_t)(row0 + c0 + t) * a.ldo + (size_t)h * a.Dv + dv0 + c] = o;
        }
        __syncthreads();
        // state: S <- a^nc S + sum_s a^(nc - 1 - s) k_s v_s^T
        for (int i = tid; i < D * DS; i += 256) {
            const int d = i / DS, c = i - d * DS;
            float sv = S[i] * pw[nc];
            for (int s = 0; s < nc; ++s) sv = fmaf(K[s * DP + d] * pw[nc - 1 - s], V[s * DS + c], sv);
            S[i] = sv;
        }
    }
    __syncthreads();
    for (int i = tid; i < D * DS; i += 256) {
        const int d = i / DS, c = i - d * DS;
        if (c < nd) Sg[(size_t)d * a.Dv + c] = S[i];
    }
}

// ---------------------------------------------------------------- linear attention over long prompts: three passes
// The walk above is sequential over a sequence's chunks.  For prompts the same result comes from three launches whose blocks
// are (chunk, sequence, head), all chunks at once:
//   1. chunk_update:  U_c = sum_s a^(n_c - 1 - s) k_s v_s^T, what chunk c adds to the state          -> ws[c]
//   2. chunk_scan:    per state element, over the chunks in order: ws[c] <- the state BEFORE chunk c, S <- a^(n_c) S + U_c;
//                     the state after the last chunk goes to the slot's array
//   3. chunk_output:  o_t = a^(t + 1) S_c^T q_t + sum_{s <= t} (q_t.k_s a^(t - s)) v_s  -- one product of [Q a^(t+1) | A]
//                     with [S_c ; V], 4 x 4 outputs per thread
// A launch covers the chunks c_begin .. c_begin + grid.x - 1 of every sequence (the host bounds the workspace by walking
// long prompts in segments; the scan picks the state up from the slot's array where the segment before left it).
struct LinChunkArgs {
    const float* proj; int ld, q_off, k_off, v_off;
    float* out; int ldo;
    float* state; const float* decay; const int4* seqs;
    int H, D, Dv, c_begin;
    float* ws;                           // [sequences][grid.x chunks][H][D][Dv]
};

__device__ __forceinline__ int round4(int n) { return (n + 3) & ~3; }

__global__ void __launch_bounds__(256) linear_chunk_update_kernel(LinChunkArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int D = a.D, Dv = a.Dv, D4 = round4(D), V4 = round4(Dv);
    float* Ks = sm;                      // [LC][D4], rows scaled by a^(nc - 1 - s)
    float* Vs = Ks + LC * D4;            // [LC][V4]
    const int4 sq = a.seqs[blockIdx.y];
    const int c = a.c_begin + blockIdx.x, h = blockIdx.z;
    if (c * LC >= sq.y) return;
    const int nc = min(LC, sq.y - c * LC), r0 = sq.x + c * LC, tid = threadIdx.x;
    const float dec = a.decay[h];
    for (int i = tid; i < LC * D4; i += 256) {
        const int s = i / D4, d = i - s * D4;
        Ks[i] = (s < nc && d < D) ? a.proj[(size_t)(r0 + s) * a.ld + a.k_off + (size_t)h * D + d] * powf(dec, (float)(nc - 1 - s)) : 0.f;
    }
    for (int i = tid; i < LC * V4; i += 256) {
        const int s = i / V4, v = i - s * V4;
        Vs[i] = (s < nc && v < Dv) ? a.proj[(size_t)(r0 + s) * a.ld + a.v_off + (size_t)h * Dv + v] : 0.f;
    }
    __syncthreads();
    float* U = a.ws + (((size_t)blockIdx.y * gridDim.x + blockIdx.x) * a.H + h) * D * Dv;
    const int nTv = V4 / 4, ntiles = (D4 / 4) * nTv;
    for (int tile = tid; tile < ntiles; tile += 256) {
        const int d0 = (tile / nTv) * 4, v0 = (tile % nTv) * 4;
        float acc[4][4] = {};
        for (int s2 = 0; s2 < nc; ++s2) {
            const float4 k4 = *(const float4*)(Ks + s2 * D4 + d0), v4 = *(const float4*)(Vs + s2 * V4 + v0);
            const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(kk[i], vv[j], acc[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (d0 + i < D && v0 + j < Dv) U[(size_t)(d0 + i) * Dv + v0 + j] = acc[i][j];
    }
}

// one thread per (sequence, head, state element)
__global__ void __launch_bounds__(256) linear_chunk_scan_kernel(LinChunkArgs a, int seg_chunks) {
    const size_t per = (size_t)a.D * a.Dv, e = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (e >= per) return;
    const int h = blockIdx.y;
    const int4 sq = a.seqs[blockIdx.z];
    const int nchunks = (sq.y + LC - 1) / LC;
    if (a.c_begin >= nchunks) return;
    const float dec = a.decay[h], dfull = powf(dec, (float)LC);
    float* Sg = a.state + ((size_t)sq.z * a.H + h) * per + e;
    float S = (sq.w > 0 || a.c_begin > 0) ? *Sg : 0.f;
    const int cend = min(nchunks, a.c_begin + seg_chunks);
    const float dlast = powf(dec, (float)(sq.y - (nchunks - 1) * LC));      // the sequence's last chunk may be short
    float* u0 = a.ws + (((size_t)blockIdx.z * seg_chunks) * a.H + h) * per + e;
    const size_t step = (size_t)a.H * per;
    constexpr int B = 8;                                                    // loads in flight per thread
    for (int c = a.c_begin; c < cend; c += B) {
        float add[B];
#pragma unroll
        for (int i = 0; i < B; ++i) add[i] = c + i < cend ? __ldcs(u0 + (size_t)(c + i - a.c_begin) * step) : 0.f;
#pragma unroll
        for (int i = 0; i < B; ++i) {
            if (c + i < cend) {
                __stcg(u0 + (size_t)(c + i - a.c_begin) * step, S);
                S = fmaf(S, c + i == nchunks - 1 ? dlast : dfull, add[i]);
            }
        }
    }
    *Sg = S;
}

__global__ void __launch_bounds__(256) linear_chunk_output_kernel(LinChunkArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int D = a.D, Dv = a.Dv, DP = D + 1, V4 = round4(Dv);
    float* Q = sm;                       // [LC][D + 1]
    float* K = Q + LC * DP;              // [LC][D + 1]
    float* Vs = K + LC * DP;             // [LC][V4]
    float* Ss = Vs + LC * V4;            // [LC][V4]: a slab of state rows
    float* A = Ss + LC * V4;             // [LC][LC + 1]
    float* pw = A + LC * (LC + 1);       // [LC + 1]
    const int4 sq = a.seqs[blockIdx.y];
    const int c = a.c_begin + blockIdx.x, h = blockIdx.z;
    if (c * LC >= sq.y) return;
    const int nc = min(LC, sq.y - c * LC), r0 = sq.x + c * LC, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float dec = a.decay[h];
    if (tid <= LC) pw[tid] = powf(dec, (float)tid);
    for (int i = tid; i < LC * D; i += 256) {
        const int r = i / D, d = i - r * D;
        const float* src = a.proj + (size_t)(r0 + r) * a.ld + (size_t)h * D + d;
        Q[r * DP + d] = r < nc ? src[a.q_off] : 0.f;
        K[r * DP + d] = r < nc ? src[a.k_off] : 0.f;
    }
    for (int i = tid; i < LC * V4; i += 256) {
        const int r = i / V4, v = i - r * V4;
        Vs[i] = (r < nc && v < Dv) ? a.proj[(size_t)(r0 + r) * a.ld + a.v_off + (size_t)h * Dv + v] : 0.f;
    }
    __syncthreads();
    {   // scores: lane = key s, the warp's four rows t = warp + 8 i share every key element
        float sc[4] = {0.f, 0.f, 0.f, 0.f};
        const float* k = K + lane * DP;
        for (int d = 0; d < D; ++d) {
            const float kv = k[d];
#pragma unroll
            for (int i = 0; i < 4; ++i) sc[i] = fmaf(Q[(warp + 8 * i) * DP + d], kv, sc[i]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int t = warp + 8 * i;
            A[t * (LC + 1) + lane] = lane <= t ? sc[i] * pw[t - lane] : 0.f;
        }
    }
    const float* Sc = a.ws + (((size_t)blockIdx.y * gridDim.x + blockIdx.x) * a.H + h) * D * Dv;
    const int nTv = V4 / 4, ntiles = (LC / 4) * nTv, rounds = (ntiles + 255) / 256;
    for (int rd = 0; rd < rounds; ++rd) {
        const int tile = rd * 256 + tid;
        const bool live = tile < ntiles;
        const int t0 = live ? (tile / nTv) * 4 : 0, v0 = live ? (tile % nTv) * 4 : 0;
        float acc[4][4] = {};
        for (int d0 = 0; d0 < D; d0 += LC) {
            __syncthreads();
            for (int i = tid; i < LC * V4; i += 256) {
                const int r = i / V4, v = i - r * V4;
                Ss[i] = (d0 + r < D && v < Dv) ? Sc[(size_t)(d0 + r) * Dv + v] : 0.f;
            }
            __syncthreads();
            if (live) {
                const int nd = min(LC, D - d0);
                for (int dd = 0; dd < nd; ++dd) {
                    const float4 s4 = *(const float4*)(Ss + dd * V4 + v0);
                    const float ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float q = Q[(t0 + i) * DP + d0 + dd];
#pragma unroll
                        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(q, ss[j], acc[i][j]);
                    }
                }
            }
        }
        if (!live) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] *= pw[t0 + i + 1];
        for (int s2 = 0; s2 < nc; ++s2) {
            const float4 v4 = *(const float4*)(Vs + s2 * V4 + v0);
            const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float w = A[(t0 + i) * (LC + 1) + s2];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(w, vv[j], acc[i][j]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (t0 + i < nc && v0 + j < Dv) a.out[(size_t)(r0 + t0 + i) * a.ldo + (size_t)h * Dv + v0 + j] = acc[i][j];
    }
}

// ---------------------------------------------------------------- linear attention: output norm and gate
struct LinFinishArgs {
    float* o; int ldo; const float* gate; int ldg, g_off;
    const float* w;                      // [H * Dv] or NULL
    int H, Dv, per_head, gate_act;       // gate_act 0 none, 1 sigmoid, 2 silu
    float eps, mult;
};

__global__ void __launch_bounds__(256) linear_finish_kernel(LinFinishArgs a) {
    __shared__ float red[8];
    __shared__ float inv_s[256];
    const int t = blockIdx.x, n = a.H * a.Dv, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* o = a.o + (size_t)t * a.ldo;
    const float* g = a.gate ? a.gate + (size_t)t * a.ldg + a.g_off : nullptr;
    if (a.per_head) {
        for (int h0 = 0; h0 < a.H; h0 += 256) {
            __syncthreads();
            for (int h = h0 + warp; h < min(a.H, h0 + 256); h += 8) {
                float ss = 0.f;
                for (int d = lane; d < a.Dv; d += 32) { const float v = o[(size_t)h * a.Dv + d]; ss = fmaf(v, v, ss); }
                ss = warp_sum(ss);
                if (lane == 0) inv_s[h - h0] = 1.f / sqrtf(ss / (float)a.Dv + a.eps);
            }
            __syncthreads();
            const int lim = min(a.H, h0 + 256) * a.Dv;
            for (int i = h0 * a.Dv + threadIdx.x; i < lim; i += 256) {
                float v = o[i] * inv_s[i / a.Dv - h0];
                if (a.w) v *= a.w[i];
                if (a.gate_act == 1) v *= sigmoid_f(g[i]); else if (a.gate_act == 2) v *= silu_f(g[i]);
                o[i] = v * a.mult;
            }
        }
        return;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) { const float v = o[i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.f / sqrtf(tot / (float)n + a.eps);
    for (int i = threadIdx.x; i < n; i += 256) {
        float v = o[i] * inv;
        if (a.w) v *= a.w[i];
        if (a.gate_act == 1) v *= sigmoid_f(g[i]); else if (a.gate_act == 2) v *= silu_f(g[i]);
        o[i] = v * a.mult;
    }
}

}  // namespace

extern "C" {

int pgk_causal_conv_rows_ex_f32(const float* h, int ldh, float* u, int ldu, const float* weight, float* state, const int32_t* slot,
                                const int32_t* pos, const int32_t* parity, int rows, int width, int taps, int residual,
                                int activation, void* stream) {
    PGK_REQUIRE(taps >= 1 && width > 0 && (taps == 1 || state), "causal_conv_rows failed: taps %d, width %d", taps, width);
    PGK_REQUIRE(h != u && ldh >= width && ldu >= width, "causal_conv_rows failed: the output rows must not be the input rows");
    PGK_REQUIRE(taps == 1 || parity || (ldh == width), "causal_conv_rows failed: strided rows need the ring kept twice");
    if (rows <= 0) return 0;
    ConvArgs a{h, u, weight, state, slot, pos, taps > 1 ? parity : nullptr, rows, width, taps, ldh, ldu, residual ? 1 : 0,
               activation ? 1 : 0};
    PGK_CUDA(launch(causal_conv_rows_kernel, dim3(rows, (width + 255) / 256), dim3(256), 0, (cudaStream_t)stream, a));
    return 0;
}

int pgk_causal_conv_rows_f32(const float* h, float* u, const float* weight, float* state, const int32_t* slot,
                             const int32_t* pos, const int32_t* parity, int rows, int width, int taps, void* stream) {
    return pgk_causal_conv_rows_ex_f32(h, width, u, width, weight, state, slot, pos, parity, rows, width, taps, 1, 0, stream);
}

int pgk_causal_conv_state_f32(const float* h, float* state, const int32_t* seqs, int n_seqs, int width, int taps, void* stream) {
    PGK_REQUIRE(taps >= 1 && width > 0, "causal_conv_state failed: taps %d, width %d", taps, width);
    if (n_seqs <= 0 || taps == 1) return 0;
    PGK_CUDA(launch(causal_conv_state_kernel, dim3(n_seqs * (taps - 1), (width + 255) / 256), dim3(256), 0, (cudaStream_t)stream,
                    h, state, (const int4*)seqs, width, taps - 1));
    return 0;
}

int pgk_seq_linear_prep(float* proj, int ld, int tokens, int heads, int dim, int vdim, int q_off, int k_off, int v_off,
                        int activation, int rot_dims, const double* inv_freq, float k_scale, const int32_t* pos, void* stream) {
    PGK_REQUIRE(heads > 0 && dim > 0 && vdim > 0, "seq_linear_prep failed: invalid head layout");
    PGK_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim && (rot_dims == 0 || inv_freq),
                "seq_linear_prep failed: %d rotated dimensions in heads of %d", rot_dims, dim);
    if (tokens <= 0 || (!activation && rot_dims == 0 && k_scale == 1.f)) return 0;
    LinPrepArgs a{proj, ld, heads, dim, vdim, q_off, k_off, v_off, activation ? 1 : 0, rot_dims, inv_freq, k_scale, pos};
    PGK_CUDA(launch(linear_prep_kernel, dim3(tokens, (3 * heads + 3) / 4), dim3(128), 0, (cudaStream_t)stream, a));
    return 0;
}

int pgk_seq_linear_value_slice(int heads, int dim, int vdim, int n_seqs) {
    // value columns per block: as narrow as fills the GPU, never below 8, and S [dim][slice] + the chunk within shared memory
    int ds = vdim;
    while (ds > 8 && (long long)n_seqs * heads * ((vdim + ds - 1) / ds) < 2 * 148) ds = (ds + 1) / 2;
    while (ds > 1 && sizeof(float) * ((size_t)dim * ds + 2 * LC * (dim + 1) + LC * ds + LC * (LC + 1) + LC + 1) > 160 * 1024) ds = (ds + 1) / 2;
    return ds;
}

int pgk_seq_linear_attention(const float* proj, int ld, int q_off, int k_off, int v_off, float* out, int ldo, float* state,
                             const float* decay, const int32_t* seqs, int n_seqs, int heads, int dim, int vdim, int value_slice,
                             void* stream) {
    PGK_REQUIRE(heads > 0 && dim > 0 && vdim > 0 && value_slice > 0, "seq_linear_attention failed: invalid head layout");
    if (n_seqs <= 0) return 0;
    const int ds = value_slice < vdim ? value_slice : vdim;
    const size_t smem = sizeof(float) * ((size_t)dim * ds + 2 * LC * (dim + 1) + LC * ds + LC * (LC + 1) + LC + 1);
    PGK_REQUIRE(smem <= 200 * 1024, "seq_linear_attention failed: heads of %d x %d need %zu bytes of shared memory", dim, ds, smem);
    static bool configured = false;
    if (smem > 40 * 1024 && !configured) {
        PGK_CUDA(cudaFuncSetAttribute(linear_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = true;
    }
    LinArgs a{proj, ld, q_off, k_off, v_off, out, ldo, state, decay, (const int4*)seqs, heads, dim, vdim, ds};
    PGK_CUDA(launch(linear_attention_kernel, dim3(n_seqs, heads, (vdim + ds - 1) / ds), dim3(256), smem, (cudaStream_t)stream, a));
    return 0;
}

int pgk_seq_linear_chunk_tokens(void) { return LC; }

int pgk_seq_linear_attention_chunks(const float* proj, int ld, int q_off, int k_off, int v_off, float* out, int ldo, float* state,
                                    const float* decay, const int32_t* seqs, int n_seqs, int heads, int dim, int vdim,
                                    int chunk_begin, int chunks, float* workspace, void* stream) {
    PGK_REQUIRE(heads > 0 && dim > 0 && vdim > 0 && chunk_begin >= 0 && workspace, "seq_linear_attention_chunks failed: invalid arguments");
    if (n_seqs <= 0 || chunks <= 0) return 0;
    const int D4 = (dim + 3) & ~3, V4 = (vdim + 3) & ~3;
    const size_t smem1 = sizeof(float) * ((size_t)LC * D4 + (size_t)LC * V4);
    const size_t smem3 = sizeof(float) * (2 * (size_t)LC * (dim + 1) + 2 * (size_t)LC * V4 + LC * (LC + 1) + LC + 1);
    PGK_REQUIRE(smem1 <= 200 * 1024 && smem3 <= 200 * 1024, "seq_linear_attention_chunks failed: heads of %d x %d need %zu bytes of shared memory", dim, vdim, smem3);
    static bool configured = false;
    if (!configured) {
        PGK_CUDA(cudaFuncSetAttribute(linear_chunk_update_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        PGK_CUDA(cudaFuncSetAttribute(linear_chunk_output_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = true;
    }
    LinChunkArgs a{proj, ld, q_off, k_off, v_off, out, ldo, state, decay, (const int4*)seqs, heads, dim, vdim, chunk_begin, workspace};
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(chunks, n_seqs, heads);
    PGK_CUDA(launch(linear_chunk_update_kernel, grid, dim3(256), smem1, st, a));
    const size_t per = (size_t)dim * vdim;
    PGK_CUDA(launch(linear_chunk_scan_kernel, dim3((unsigned)((per + 255) / 256), heads, n_seqs), dim3(256), 0, st, a, chunks));
    PGK_CUDA(launch(linear_chunk_output_kernel, grid, dim3(256), smem3, st, a));
    return 0;
}

int pgk_seq_linear_finish(float* o, int ldo, const float* gate_rows, int ldg, int gate_off, const float* weight, int tokens,
                          int heads, int vdim, int per_head, int gate_act, float eps, float mult, void* stream) {
    PGK_REQUIRE(heads > 0 && vdim > 0 && gate_act >= 0 && gate_act <= 2 && (gate_act == 0 || gate_rows),
                "seq_linear_finish failed: invalid arguments");
    if (tokens <= 0) return 0;
    LinFinishArgs a{o, ldo, gate_rows, ldg, gate_off, weight, heads, vdim, per_head ? 1 : 0, gate_act, eps, mult};
    PGK_CUDA(launch(linear_finish_kernel, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, a));
    return 0;
}

}  // extern "C"
