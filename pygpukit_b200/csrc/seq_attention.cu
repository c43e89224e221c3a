// seq_attention.cu -- attention over a paged key/value cache for ragged batches (any mix of prompt portions and single
// decoded tokens), float32 arithmetic throughout.
//
// Cache: pages of PS positions; page p of a layer holds K rows [G][PS][D] and V rows [G][PS][Dv] in bfloat16 or float32;
// `table` [slots][max_pages] maps (sequence slot, position / PS) to a page.
//
//   mixer_prep:  per token, on the fused projection row [q | k | v | gate]: RMS norm of every query head (in place) and
//                key head (weights shared by the heads), optional value mixing v <- (1 - lam) v + lam v_first (or recording
//                v as v_first), K and V rows written to the cache at the token's position.
//   attention:   score = scale q.k -> cap tanh(score / cap) -> minus slope_h (i - j); key j is visible from query i when
//                j <= i and, with a chunk size C, floor(j / C) == floor(i / C); online softmax; P.V; optional output gate
//                out *= sigmoid(gate).  A block serves one tile of consecutive queries of one sequence and one KV head
//                (all query heads of its group), K/V tiles of 32 positions staged in shared memory, a lane per key.
//                Optional: a sliding window (key j visible when i - j < window), a sink per head (a score that enters the
//                softmax denominator once and has no value: the running (max, sum) starts at (sink, 1) instead of
//                (-inf, 0)), a gate of one number per head, values that are a prefix of the key rows (latent attention:
//                one cache array, no second staging), and row strides of the cache rows.
//   mixer_prep_all: the form whose q / k norm runs over the WHOLE projection (all heads at once), with projection
//                biases and values that are the keys before the norm.
#include "common.cuh"
#include "../../include/pgk_b200.h"

using namespace pgk;

namespace {

template <typename TC> __device__ __forceinline__ float cload(const TC* p);
template <> __device__ __forceinline__ float cload<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float cload<uint16_t>(const uint16_t* p) { return bf16_bits_to_f32(*p); }
template <typename TC> __device__ __forceinline__ void cstore(TC* p, float v);
template <> __device__ __forceinline__ void cstore<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void cstore<uint16_t>(uint16_t* p, float v) { *p = f32_to_bf16_bits(v); }

struct PrepArgs {
    float* proj; int ld;
    int H, G, D, Dv;
    const float* qw; const float* kw; float eps;
    int vmode; float lam; float* vfirst;            // 0: none, 1: record v, 2: mix with the recorded v
    void* kc; void* vc; const int* table; int max_pages, PS;
    const int* slot; const int* pos;
};

// units: H query heads, G key heads, G value heads; one warp each, four per block
template <typename TC>
__global__ void __launch_bounds__(128) mixer_prep_kernel(PrepArgs a) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int u = blockIdx.y * 4 + warp;
    if (u >= a.H + 2 * a.G) return;
    float* row = a.proj + (size_t)t * a.ld;
    const int pos = a.pos[t], slot = a.slot[t];
    const int page = a.table[(size_t)slot * a.max_pages + pos / a.PS], r = pos % a.PS;
    if (u < a.H + a.G) {
        float* x = row + (size_t)u * a.D;            // query heads then key heads are contiguous
        float ss = 0.f;
        for (int d = lane; d < a.D; d += 32) ss = fmaf(x[d], x[d], ss);
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss / (float)a.D + a.eps);
        if (u < a.H) {
            for (int d = lane; d < a.D; d += 32) x[d] = x[d] * inv * a.qw[d];
        } else {
            const int g = u - a.H;
            TC* dst = (TC*)a.kc + (((size_t)page * a.G + g) * a.PS + r) * a.D;
            for (int d = lane; d < a.D; d += 32) cstore<TC>(dst + d, x[d] * inv * a.kw[d]);
        }
        return;
    }
    const int g = u - a.H - a.G, GV = a.G * a.Dv;
    const int voff = a.H * a.D + a.G * a.D + g * a.Dv;
    TC* dst = (TC*)a.vc + (((size_t)page * a.G + g) * a.PS + r) * a.Dv;
    for (int d = lane; d < a.Dv; d += 32) {
        float v = row[voff + d];
        if (a.vmode == 1) a.vfirst[(size_t)t * GV + g * a.Dv + d] = v;
        else if (a.vmode == 2) v = (1.f - a.lam) * v + a.lam * a.vfirst[(size_t)t * GV + g * a.Dv + d];
        cstore<TC>(dst + d, v);
    }
}

struct PrepRotArgs {
    float* proj; int ld;
    int H, G, D, Dv, q_off, k_off, v_off;
    int rot_dims; const double* inv_freq;
    int norm;                                        // 0: none, 1: divide by the root mean square, 2: and multiply by qw / kw
    const float* qw; const float* kw; float eps;
    void* kc; void* vc; const int* table; int max_pages, PS;
    const int* slot; const int* pos;
    const float* qb; const float* kb; const float* vb;      // projection biases [H x D], [G x D], [G x Dv] or NULL
    const float* q_mult;                                     // [H] factor on every query head (a per-head temperature) or NULL
};

// units: H query heads (rotated and normalised in place), G key heads and G value heads (into the cache); a warp each.
// Rotation: element i < rot_dims / 2 of a head is paired with element i + rot_dims / 2, angle = position * inv_freq[i].
template <typename TC>
__global__ void __launch_bounds__(128) mixer_prep_rot_kernel(PrepRotArgs a) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int u = blockIdx.y * 4 + warp;
    if (u >= a.H + 2 * a.G) return;
    float* row = a.proj + (size_t)t * a.ld;
    const int pos = a.pos[t], slot = a.slot[t];
    const int page = a.table[(size_t)slot * a.max_pages + pos / a.PS], r = pos % a.PS;
    if (u >= a.H + a.G) {
        const int g = u - a.H - a.G;
        const float* v = row + a.v_off + (size_t)g * a.Dv;
        TC* dst = (TC*)a.vc + (((size_t)page * a.G + g) * a.PS + r) * a.Dv;
        const float* vb = a.vb ? a.vb + (size_t)g * a.Dv : nullptr;
        for (int d = lane; d < a.Dv; d += 32) cstore<TC>(dst + d, v[d] + (vb ? vb[d] : 0.f));
        return;
    }
    const bool is_k = u >= a.H;
    const int g = u - a.H;
    float* x = row + (is_k ? a.k_off + (size_t)g * a.D : a.q_off + (size_t)u * a.D);
    const float* bias = is_k ? (a.kb ? a.kb + (size_t)g * a.D : nullptr) : (a.qb ? a.qb + (size_t)u * a.D : nullptr);
    const float qm = (!is_k && a.q_mult) ? a.q_mult[u] : 1.f;
    if (!is_k && a.rot_dims == 0 && a.norm == 0 && !bias && !a.q_mult) return;      // the query stays as projected
    const int half = a.rot_dims / 2;
    float ss = 0.f;
    for (int i = lane; i < half; i += 32) {
        float sn, cs;
        rope_angle_sincos(pos, a.inv_freq[i], sn, cs);
        const float p0 = x[i] + (bias ? bias[i] : 0.f), p1 = x[i + half] + (bias ? bias[i + half] : 0.f);
        const float r0 = p0 * cs - p1 * sn, r1 = p1 * cs + p0 * sn;
        x[i] = r0; x[i + half] = r1;
        ss = fmaf(r0, r0, fmaf(r1, r1, ss));
    }
    for (int d = 2 * half + lane; d < a.D; d += 32) {
        const float v = x[d] + (bias ? bias[d] : 0.f);
        if (bias) x[d] = v;
        ss = fmaf(v, v, ss);
    }
    __syncwarp();
    float inv = 1.f;
    if (a.norm) inv = 1.f / sqrtf(warp_sum(ss) / (float)a.D + a.eps);
    const float* w = a.norm == 2 ? (is_k ? a.kw : a.qw) : nullptr;
    if (is_k) {
        TC* dst = (TC*)a.kc + (((size_t)page * a.G + g) * a.PS + r) * a.D;
        for (int d = lane; d < a.D; d += 32) cstore<TC>(dst + d, x[d] * inv * (w ? w[d] : 1.f));
    } else if (a.norm || a.q_mult) {
        for (int d = lane; d < a.D; d += 32) x[d] = x[d] * inv * (w ? w[d] : 1.f) * qm;
    }
}

struct PrepAllArgs {
    float* proj; int ld;
    int H, G, D, k_off;
    const float* qb; const float* kb; const float* qw; const float* kw; float w_off, eps;
    void* kc; void* vc; const int* table; int max_pages, PS;
    const int* slot; const int* pos;
};

__device__ __forceinline__ float block_sum_256(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += red[i];
    return s;
}

// one block per token: q <- (q + b_q) / rms(all of q) * (w_off + w_q) in place; the cache gets (k + b_k) as the VALUE row and
// (k + b_k) / rms(all of k) * (w_off + w_k) as the KEY row, head by head
template <typename TC>
__global__ void __launch_bounds__(256) mixer_prep_all_kernel(PrepAllArgs a) {
    __shared__ float red[8];
    const int t = blockIdx.x;
    float* q = a.proj + (size_t)t * a.ld;
    float* k = q + a.k_off;
    const int nq = a.H * a.D, nk = a.G * a.D;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
        const float v = q[i] + (a.qb ? a.qb[i] : 0.f);
        q[i] = v;
        sq = fmaf(v, v, sq);
    }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        const float v = k[i] + (a.kb ? a.kb[i] : 0.f);
        k[i] = v;
        sk = fmaf(v, v, sk);
    }
    sq = block_sum_256(sq, red);
    sk = block_sum_256(sk, red);
    const float iq = 1.f / sqrtf(sq / (float)nq + a.eps), ik = 1.f / sqrtf(sk / (float)nk + a.eps);
    for (int i = threadIdx.x; i < nq; i += blockDim.x) q[i] = q[i] * iq * (a.w_off + a.qw[i]);
    const int pos = a.pos[t], slot = a.slot[t];
    const int page = a.table[(size_t)slot * a.max_pages + pos / a.PS], r = pos % a.PS;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        const int g = i / a.D, d = i - g * a.D;
        const size_t o = (((size_t)page * a.G + g) * a.PS + r) * a.D + d;
        const float v = k[i];
        cstore<TC>((TC*)a.vc + o, v);
        cstore<TC>((TC*)a.kc + o, v * ik * (a.w_off + a.kw[i]));
    }
}

struct AttnArgs {
    const float* proj; int ld, q_off, g_off;
    float* out; int ldo;
    const void* kc; const void* vc; const int* table; int max_pages, PS;
    const float* gsrc; int ldg;         // rows the gate is read from (gate 1: g_off + h * Dv + dv, gate 2: g_off + h)
    const float* sinks;                 // [H] or NULL: a score per head that joins the denominator and has no value
    int window;                         // > 0: key j is visible from i only when i - j < window
    int kld, vld;                       // elements between consecutive positions' rows in the K / V arrays
    int valias;                         // the value rows are the first Dv elements of the key rows (one staging)
    const int4* tiles;                  // (first token row, queries, slot, first position)
    const float* slopes;                // [H] or NULL
    const float* slopes2;               // [H] or NULL: the distance term is slopes[h] * ln(1 + slopes2[h] * (i - j)) instead
    int keep;                           // with a window: the first `keep` positions stay visible beyond it
    int prob;                           // 0: softmax over the visible keys; 1: weight sigmoid(score + pbias[h]), not normalised
    const float* pbias;                 // [H] or NULL
    float out_mult;                     // constant factor on the output
    int H, G, D, Dv, chunk, HB, gate;
    float scale, cap;
    int splits; float* ws;              // splits > 1: partial (m, l, acc[Dv]) records [row][H][splits][Dv + 2]
    unsigned* tickets;                  // one arrival counter per (tile, head block), zero between launches
};

constexpr int KT = 32;                  // keys per tile = one per lane

__device__ __forceinline__ float gate_logit(const AttnArgs& a, size_t t, int h, int dv) {
    return a.gsrc[t * a.ldg + a.g_off + (a.gate == 2 ? (size_t)h : (size_t)h * a.Dv + dv)];
}
__device__ __forceinline__ int first_key(const AttnArgs& a, int pos) {
    int lo = a.chunk > 0 ? (pos / a.chunk) * a.chunk : 0;
    if (a.window > 0) lo = max(lo, pos - a.window + 1);
    return lo;
}
// The keys of a tile whose lowest window start is jlo come in two runs: the kept first positions below jlo, [0, kept), and
// [jlo, jhi].  Key tile ti covers KT positions from tile_first(); positions past tile_last() are padding.
__device__ __forceinline__ int kept_below(const AttnArgs& a, int jlo) { return a.window > 0 ? min(a.keep, jlo) : 0; }
__device__ __forceinline__ float distance_term(float slope, float slope2, bool log_form, int dist) {
    const float d = (float)max(dist, 0);
    return log_form ? slope * log1pf(slope2 * d) : slope * d;
}

// KT cache rows of n elements -> shared memory as float32 (row stride ld), 16 bytes per load when the rows allow it;
// rows with offset < 0 (past the last key) are zero-filled
template <typename TC>
__device__ __forceinline__ void stage_rows(float* dst, int ld, const TC* base, const long long* row_off, int n, int src_ld) {
    constexpr int VEC = 16 / sizeof(TC);
    if (n % VEC == 0 && src_ld % VEC == 0) {
        const int vpr = n / VEC;
#pragma unroll 2
        for (int i = threadIdx.x; i < KT * vpr; i += blockDim.x) {
            const int r = i / vpr, c = (i - r * vpr) * VEC;
            float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (row_off[r] >= 0) {
                const uint4 v = *(const uint4*)(base + row_off[r] + c);
                if (sizeof(TC) == 2) {
                    f[0] = bf16lo(v.x); f[1] = bf16hi(v.x); f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
                    f[4] = bf16lo(v.z); f[5] = bf16hi(v.z); f[6] = bf16lo(v.w); f[7] = bf16hi(v.w);
                } else {
                    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
                }
            }
#pragma unroll
            for (int q = 0; q < VEC; ++q) dst[r * ld + c + q] = f[q];
        }
        return;
    }
    for (int i = threadIdx.x; i < KT * n; i += blockDim.x) {
        const int r = i / n, d = i - r * n;
        dst[r * ld + d] = row_off[r] >= 0 ? cload<TC>(base + row_off[r] + d) : 0.f;
    }
}
constexpr int PPW = 4;                  // (query, head) pairs per warp
constexpr int NWARP = 8;

template <typename TC, int NV>
__global__ void __launch_bounds__(256) seq_attention_kernel(AttnArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int D = a.D, Dv = a.Dv, DP = D + 1;
    float* qs = sm;                                   // [NWARP][D][PPW]
    float* Ks = qs + NWARP * D * PPW;                 // [KT][D + 1]
    float* Vs = a.valias ? Ks : Ks + KT * DP;         // [KT][Dv] (the key rows themselves when the values alias them)
    const int vstr = a.valias ? DP : Dv;
    __shared__ long long krow[KT], vrow[KT];

    const int4 tile = a.tiles[blockIdx.x];
    const int t0 = tile.x, nq = tile.y, slot = tile.z, pos0 = tile.w;
    const int rep = a.H / a.G, hsplit = (rep + a.HB - 1) / a.HB;
    const int g = blockIdx.y / hsplit, hpart = blockIdx.y - g * hsplit;
    const int hb0 = g * rep + hpart * a.HB, nh = min(a.HB, rep - hpart * a.HB);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // this warp's pairs
    int qi[PPW], hd[PPW], pi[PPW], lo[PPW];
    bool ok[PPW];
    float slope[PPW], slope2[PPW], pb[PPW];
    const bool log_form = a.slopes2 != nullptr;
#pragma unroll
    for (int c = 0; c < PPW; ++c) {
        const int p = warp * PPW + c;
        qi[c] = p / a.HB;
        const int hh = p - qi[c] * a.HB;
        ok[c] = qi[c] < nq && hh < nh;
        hd[c] = hb0 + hh;
        pi[c] = pos0 + qi[c];
        lo[c] = first_key(a, pi[c]);
        slope[c] = (ok[c] && a.slopes) ? a.slopes[hd[c]] : 0.f;
        slope2[c] = (ok[c] && a.slopes2) ? a.slopes2[hd[c]] : 0.f;
        pb[c] = (ok[c] && a.pbias) ? a.pbias[hd[c]] : 0.f;
    }
    const bool warp_live = ok[0] || ok[1] || ok[2] || ok[3];
    for (int i = lane; i < D * PPW; i += 32) {
        const int d = i / PPW, c = i - d * PPW;
        float v = 0.f;
#pragma unroll
        for (int cc = 0; cc < PPW; ++cc)
            if (cc == c && ok[cc]) v = a.proj[(size_t)(t0 + qi[cc]) * a.ld + a.q_off + (size_t)hd[cc] * D + d];
        qs[(warp * D + d) * PPW + c] = v;
    }
    float m[PPW], l[PPW], acc[PPW][NV];
#pragma unroll
    for (int c = 0; c < PPW; ++c) {
        m[c] = -INFINITY; l[c] = 0.f;
        if (a.sinks && ok[c] && blockIdx.z == 0) { m[c] = a.sinks[hd[c]]; l[c] = 1.f; }    // the sink counts once: slice 0
        if (a.prob) { m[c] = 0.f; l[c] = blockIdx.z == 0 ? 1.f : 0.f; }                    // plain sums: the slices' weights are 1
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[c][v] = 0.f;
    }
    const int jlo = first_key(a, pos0), jhi = pos0 + nq - 1;
    const TC* kc = (const TC*)a.kc;
    const TC* vc = (const TC*)a.vc;
    // this block's slice of the key tiles (all of them when splits == 1)
    const int kept = kept_below(a, jlo), nkept = (kept + KT - 1) / KT;
    const int ntile = nkept + (jhi - jlo) / KT + 1, per = (ntile + a.splits - 1) / a.splits;
    const int tbeg = (int)blockIdx.z * per, tend = min(ntile, tbeg + per);
    for (int ti = tbeg; ti < tend; ++ti) {
        const int j0 = ti < nkept ? ti * KT : jlo + (ti - nkept) * KT;
        const int jmax = ti < nkept ? kept - 1 : jhi;
        __syncthreads();
        if (threadIdx.x < KT) {
            const int j = j0 + threadIdx.x;
            long long ko = -1, vo = -1;
            if (j <= jmax) {
                const int page = a.table[(size_t)slot * a.max_pages + j / a.PS], r = j % a.PS;
                ko = (((long long)page * a.G + g) * a.PS + r) * a.kld;
                vo = (((long long)page * a.G + g) * a.PS + r) * a.vld;
            }
            krow[threadIdx.x] = ko; vrow[threadIdx.x] = vo;
        }
        __syncthreads();
        stage_rows<TC>(Ks, DP, kc, krow, D, a.kld);
        if (!a.valias) stage_rows<TC>(Vs, Dv, vc, vrow, Dv, a.vld);
        __syncthreads();
        if (!warp_live) continue;                   // a warp without a (query, head) pair only helps staging
        // scores: lane = key
        float s[PPW] = {};
        const float* kr = Ks + lane * DP;
        const float4* q4 = (const float4*)(qs + warp * D * PPW);
        for (int d = 0; d < D; ++d) {
            const float kv = kr[d];
            const float4 q = q4[d];
            s[0] = fmaf(q.x, kv, s[0]); s[1] = fmaf(q.y, kv, s[1]);
            s[2] = fmaf(q.z, kv, s[2]); s[3] = fmaf(q.w, kv, s[3]);
        }
        const int j = j0 + lane;
        float p[PPW];
#pragma unroll
        for (int c = 0; c < PPW; ++c) {
            float sc = s[c] * a.scale;
            if (a.cap > 0.f) sc = a.cap * tanhf(sc / a.cap);
            sc -= distance_term(slope[c], slope2[c], log_form, pi[c] - j);
            const bool vis = ok[c] && j <= jmax && j <= pi[c] && (j >= lo[c] || j < a.keep);
            if (a.prob) { p[c] = vis ? 1.f / (1.f + expf(-(sc + pb[c]))) : 0.f; continue; }
            sc = vis ? sc : -INFINITY;
            const float mn = fmaxf(m[c], warp_max(sc));
            if (mn == -INFINITY) { p[c] = 0.f; continue; }      // uniform across the warp
            const float corr = expf(m[c] - mn);
            p[c] = expf(sc - mn);
            l[c] = l[c] * corr + warp_sum(p[c]);
            m[c] = mn;
#pragma unroll
            for (int v = 0; v < NV; ++v) acc[c][v] *= corr;
        }
        const int nvalid = min(KT, jmax - j0 + 1);
        for (int jj = 0; jj < nvalid; ++jj) {
            float pj[PPW];
#pragma unroll
            for (int c = 0; c < PPW; ++c) pj[c] = __shfl_sync(0xffffffffu, p[c], jj);
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                const int dv = lane + 32 * v;
                const float vv = dv < Dv ? Vs[jj * vstr + dv] : 0.f;
#pragma unroll
                for (int c = 0; c < PPW; ++c) acc[c][v] = fmaf(pj[c], vv, acc[c][v]);
            }
        }
    }
    if (a.splits > 1) {
        // every slice leaves (max, sum, P.V) records; the block that arrives last folds them (threadfence + ticket)
#pragma unroll
        for (int c = 0; c < PPW; ++c) {
            if (!ok[c]) continue;
            float* rec = a.ws + (((size_t)(t0 + qi[c]) * a.H + hd[c]) * a.splits + blockIdx.z) * (Dv + 2);
            if (lane == 0) { rec[0] = m[c]; rec[1] = l[c]; }
#pragma unroll
            for (int v = 0; v < NV; ++v)
                if (lane + 32 * v < Dv) rec[2 + lane + 32 * v] = acc[c][v];
        }
        __shared__ unsigned last;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned* tk = a.tickets + (size_t)blockIdx.x * gridDim.y + blockIdx.y;
            const unsigned n = atomicAdd(tk, 1u);
            last = (n == (unsigned)a.splits - 1u);
            if (last) *tk = 0u;
        }
        __syncthreads();
        if (!last) return;
        __threadfence();
        // fold, phase 1: per pair the slices' weights exp(m_s - M) / L (lanes over slices)
        __shared__ float wsl[NWARP * PPW][64];
#pragma unroll
        for (int c = 0; c < PPW; ++c) {
            if (!ok[c]) continue;
            const float* rec = a.ws + (((size_t)(t0 + qi[c]) * a.H + hd[c]) * a.splits) * (Dv + 2);
            float ms[2], ls[2], M = -INFINITY;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int sp = lane + 32 * u;
                ms[u] = sp < a.splits ? __ldcg(rec + (size_t)sp * (Dv + 2)) : -INFINITY;
                ls[u] = sp < a.splits ? __ldcg(rec + (size_t)sp * (Dv + 2) + 1) : 0.f;
                M = fmaxf(M, ms[u]);
            }
            M = warp_max(M);
            float e[2], L = 0.f;
#pragma unroll
            for (int u = 0; u < 2; ++u) { e[u] = ms[u] == -INFINITY ? 0.f : expf(ms[u] - M); L += ls[u] * e[u]; }
            L = warp_sum(L);
            const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
            for (int u = 0; u < 2; ++u)
                if (lane + 32 * u < a.splits) wsl[warp * PPW + c][lane + 32 * u] = e[u] * inv;
        }
        __syncthreads();
        // phase 2: every thread of the block takes outputs (pair, dv); the slices' loads are independent
        for (int i = threadIdx.x; i < NWARP * PPW * Dv; i += blockDim.x) {
            const int p = i / Dv, dv = i - p * Dv;
            const int q = p / a.HB, hh = p - q * a.HB;
            if (q >= nq || hh >= nh) continue;
            const size_t t = t0 + q;
            const int h = hb0 + hh;
            const float* rec = a.ws + ((t * a.H + h) * a.splits) * (Dv + 2) + 2 + dv;
            float o = 0.f;
#pragma unroll 8
            for (int sp = 0; sp < a.splits; ++sp) o = fmaf(wsl[p][sp], __ldcg(rec + (size_t)sp * (Dv + 2)), o);
            if (a.gate) o *= 1.f / (1.f + expf(-gate_logit(a, t, h, dv)));
            a.out[t * a.ldo + (size_t)h * Dv + dv] = o * a.out_mult;
        }
        return;
    }
#pragma unroll
    for (int c = 0; c < PPW; ++c) {
        if (!ok[c]) continue;
        const size_t t = t0 + qi[c];
        const float inv = l[c] > 0.f ? 1.f / l[c] : 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int dv = lane + 32 * v;
            if (dv >= Dv) continue;
            float o = acc[c][v] * inv;
            if (a.gate) o *= 1.f / (1.f + expf(-gate_logit(a, t, hd[c], dv)));
            a.out[t * a.ldo + (size_t)hd[c] * Dv + dv] = o * a.out_mult;
        }
    }
}

template <typename TC, int NV>
int launch_attn(const AttnArgs& a, int tiles, cudaStream_t st) {
    const size_t smem = sizeof(float) * ((size_t)NWARP * a.D * PPW + (size_t)KT * (a.D + 1) + (a.valias ? 0 : (size_t)KT * a.Dv));
    PGK_REQUIRE(smem <= 200 * 1024, "seq_attention failed: head sizes %d / %d need %zu bytes of shared memory", a.D, a.Dv, smem);
    static size_t configured = 0;
    // the opt-in is needed once dynamic + STATIC shared memory (row offsets, the fold's slice weights: ~9 KB) pass 48 KB
    if (smem > 32 * 1024 && configured == 0) {
        PGK_CUDA(cudaFuncSetAttribute(seq_attention_kernel<TC, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = 1;
    }
    const int rep = a.H / a.G, hsplit = (rep + a.HB - 1) / a.HB;
    PGK_CUDA(launch(seq_attention_kernel<TC, NV>, dim3(tiles, a.G * hsplit, a.splits), dim3(256), smem, st, a));
    return 0;
}

template <typename TC>
int launch_attn_nv(const AttnArgs& a, int tiles, cudaStream_t st) {
    const int nv = (a.Dv + 31) / 32;
    if (nv <= 1) return launch_attn<TC, 1>(a, tiles, st);
    if (nv <= 2) return launch_attn<TC, 2>(a, tiles, st);
    if (nv <= 4) return launch_attn<TC, 4>(a, tiles, st);
    if (nv <= 8) return launch_attn<TC, 8>(a, tiles, st);
    if (nv <= 16) return launch_attn<TC, 16>(a, tiles, st);
    set_error("seq_attention failed: value size %d exceeds 512", a.Dv);
    return 1;
}


// ---------------------------------------------------------------- decoding: one query per tile
// A tile holds ONE query; its (at most DPAIRS = 8 or 2) heads of the KV group are served by every warp.  No shared-memory K/V
// tiles and no block barrier in the key loop: a warp takes 32 keys at a time (a lane per key, the key's row read from the
// cache with 16-byte loads, q broadcast from shared memory), keeps its own online-softmax state for all heads, and reads
// the V rows coalesced (a lane owns NV consecutive value columns).  The eight warps' states are folded through shared
// memory; with key slices (grid.z) the block leaves one record per head and the last-arriving block folds the slices.
constexpr int DPAIRS_MAX = 8;

template <typename TC, int NV>
__device__ __forceinline__ void load_values(const TC* p, bool vec, int n_left, float (&out)[NV]) {
    if (vec) {
        if constexpr (sizeof(TC) * NV > 16) {
            constexpr int PER = 16 / sizeof(TC);
#pragma unroll
            for (int i = 0; i < NV / PER; ++i) {
                const uint4 v = *(const uint4*)(p + i * PER);
                float* o = out + i * PER;
                if constexpr (sizeof(TC) == 2) {
                    o[0] = bf16lo(v.x); o[1] = bf16hi(v.x); o[2] = bf16lo(v.y); o[3] = bf16hi(v.y);
                    o[4] = bf16lo(v.z); o[5] = bf16hi(v.z); o[6] = bf16lo(v.w); o[7] = bf16hi(v.w);
                } else {
                    o[0] = __uint_as_float(v.x); o[1] = __uint_as_float(v.y); o[2] = __uint_as_float(v.z); o[3] = __uint_as_float(v.w);
                }
            }
            return;
        } else if constexpr (sizeof(TC) * NV == 16) {
            const uint4 v = *(const uint4*)p;
            if constexpr (sizeof(TC) == 2) {
                out[0] = bf16lo(v.x); out[1] = bf16hi(v.x); out[2] = bf16lo(v.y); out[3] = bf16hi(v.y);
                out[4] = bf16lo(v.z); out[5] = bf16hi(v.z); out[6] = bf16lo(v.w); out[7] = bf16hi(v.w);
            } else {
                out[0] = __uint_as_float(v.x); out[1] = __uint_as_float(v.y); out[2] = __uint_as_float(v.z); out[3] = __uint_as_float(v.w);
            }
            return;
        } else if constexpr (sizeof(TC) * NV == 8) {
            const uint2 v = *(const uint2*)p;
            if constexpr (sizeof(TC) == 2) { out[0] = bf16lo(v.x); out[1] = bf16hi(v.x); out[2] = bf16lo(v.y); out[3] = bf16hi(v.y); }
            else { out[0] = __uint_as_float(v.x); out[1] = __uint_as_float(v.y); }
            return;
        } else if constexpr (sizeof(TC) * NV == 4 && sizeof(TC) == 2) {
            const uint32_t v = *(const uint32_t*)p;
            out[0] = bf16lo(v); out[1] = bf16hi(v);
            return;
        }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) out[i] = i < n_left ? cload<TC>(p + i) : 0.f;
}

template <typename TC, int NV, int DPAIRS>
__global__ void __launch_bounds__(256) seq_attention_decode_kernel(AttnArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int D = a.D, Dv = a.Dv;
    float* qs = sm;                                    // [DPAIRS][D]
    float* st_m = qs + DPAIRS * D;                     // [NWARP][DPAIRS]
    float* st_l = st_m + NWARP * DPAIRS;               // [NWARP][DPAIRS]
    float* st_acc = st_l + NWARP * DPAIRS;             // [NWARP][DPAIRS][Dv]

    const int4 tile = a.tiles[blockIdx.x];
    const int t0 = tile.x, slot = tile.z, pos = tile.w;
    const int rep = a.H / a.G, hsplit = (rep + DPAIRS - 1) / DPAIRS;
    const int g = blockIdx.y / hsplit, hpart = blockIdx.y - g * hsplit;
    const int hb0 = g * rep + hpart * DPAIRS, nh = min(DPAIRS, rep - hpart * DPAIRS);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // loads that depend on nothing but the tile go out first: the gate values of this thread's outputs (used last) ...
    constexpr int GPT = 4;                                // outputs (head, column) per thread kept in registers
    float gz[GPT];
#pragma unroll
    for (int u = 0; u < GPT; ++u) {
        const int i = threadIdx.x + u * 256;
        gz[u] = (a.gate && i < nh * Dv) ? gate_logit(a, (size_t)t0, hb0 + i / Dv, i % Dv) : 0.f;
    }
    for (int i = threadIdx.x; i < DPAIRS * D; i += blockDim.x) {
        const int p = i / D, d = i - p * D;
        qs[i] = p < nh ? a.proj[(size_t)t0 * a.ld + a.q_off + (size_t)(hb0 + p) * D + d] : 0.f;
    }
    float slope[DPAIRS], slope2[DPAIRS], pb[DPAIRS];
    const bool log_form = a.slopes2 != nullptr;
#pragma unroll
    for (int p = 0; p < DPAIRS; ++p) {
        slope[p] = (p < nh && a.slopes) ? a.slopes[hb0 + p] : 0.f;
        slope2[p] = (p < nh && a.slopes2) ? a.slopes2[hb0 + p] : 0.f;
        pb[p] = (p < nh && a.pbias) ? a.pbias[hb0 + p] : 0.f;
    }
    // ... and the page of the warp's first key tile
    const int jlo = first_key(a, pos), jhi = pos;
    const int kept = kept_below(a, jlo), nkept = (kept + KT - 1) / KT;
    const int ntile = nkept + (jhi - jlo) / KT + 1, per = (ntile + a.splits - 1) / a.splits;
    const int tb = (int)blockIdx.z * per, te = min(ntile, tb + per);
    int page_first = 0;
    {
        const int ti = tb + warp;
        const int j = (ti < nkept ? ti * KT : jlo + (ti - nkept) * KT) + lane;
        if (ti < te && j <= (ti < nkept ? kept - 1 : jhi)) page_first = a.table[(size_t)slot * a.max_pages + j / a.PS];
    }
    __syncthreads();

    float m[DPAIRS], l[DPAIRS], acc[DPAIRS][NV];
#pragma unroll
    for (int p = 0; p < DPAIRS; ++p) {
        m[p] = -INFINITY; l[p] = 0.f;
        if (a.sinks && p < nh && warp == 0 && blockIdx.z == 0) { m[p] = a.sinks[hb0 + p]; l[p] = 1.f; }   // counted once
        if (a.prob) { m[p] = 0.f; l[p] = (warp == 0 && blockIdx.z == 0) ? 1.f : 0.f; }                   // plain sums
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[p][v] = 0.f;
    }
    const TC* kc = (const TC*)a.kc;
    const TC* vc = (const TC*)a.vc;
    constexpr int KV = 16 / sizeof(TC);
    constexpr int VR = NV >= 16 ? 4 : 8;               // value rows in flight
    const bool kvec = D % KV == 0 && a.kld % KV == 0;
    const bool vvec = Dv % NV == 0 && a.vld % NV == 0 && (NV * (int)sizeof(TC) <= 16 || a.vld % KV == 0);
    for (int ti = tb + warp; ti < te; ti += NWARP) {
        const int j0 = ti < nkept ? ti * KT : jlo + (ti - nkept) * KT, jmax = ti < nkept ? kept - 1 : jhi;
        const int j = j0 + lane;
        const bool in = j <= jmax;
        long long ko = 0, vo = 0;
        if (in) {
            const int page = ti == tb + warp ? page_first : a.table[(size_t)slot * a.max_pages + j / a.PS], r = j % a.PS;
            ko = (((long long)page * a.G + g) * a.PS + r) * a.kld;
            vo = (((long long)page * a.G + g) * a.PS + r) * a.vld;
        }
        float s[DPAIRS];
#pragma unroll
        for (int p = 0; p < DPAIRS; ++p) s[p] = 0.f;
        if (in) {
            if (kvec) {
                for (int d0 = 0; d0 < D; d0 += 4 * KV) {          // four 16-byte loads of the key's row in flight
                    uint4 raw[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (d0 + u * KV < D) raw[u] = *(const uint4*)(kc + ko + d0 + u * KV);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int d = d0 + u * KV;
                        if (d >= D) break;
                        const uint4 v = raw[u];
                        float kf[8];
                        if (sizeof(TC) == 2) {
                            kf[0] = bf16lo(v.x); kf[1] = bf16hi(v.x); kf[2] = bf16lo(v.y); kf[3] = bf16hi(v.y);
                            kf[4] = bf16lo(v.z); kf[5] = bf16hi(v.z); kf[6] = bf16lo(v.w); kf[7] = bf16hi(v.w);
                        } else {
                            kf[0] = __uint_as_float(v.x); kf[1] = __uint_as_float(v.y); kf[2] = __uint_as_float(v.z); kf[3] = __uint_as_float(v.w);
                        }
#pragma unroll
                        for (int p = 0; p < DPAIRS; ++p) {
                            float qf[8];
                            *(float4*)&qf[0] = *(const float4*)(qs + p * D + d);
                            if (KV == 8) *(float4*)&qf[4] = *(const float4*)(qs + p * D + d + 4);
#pragma unroll
                            for (int e = 0; e < KV; ++e) s[p] = fmaf(qf[e], kf[e], s[p]);
                        }
                    }
                }
            } else {
                for (int d = 0; d < D; ++d) {
                    const float kv = cload<TC>(kc + ko + d);
#pragma unroll
                    for (int p = 0; p < DPAIRS; ++p) s[p] = fmaf(qs[p * D + d], kv, s[p]);
                }
            }
        }
        float pr[DPAIRS];
#pragma unroll
        for (int p = 0; p < DPAIRS; ++p) {
            float sc = s[p] * a.scale;
            if (a.cap > 0.f) sc = a.cap * tanhf(sc / a.cap);
            sc -= distance_term(slope[p], slope2[p], log_form, pos - j);
            if (a.prob) { pr[p] = (in && p < nh) ? 1.f / (1.f + expf(-(sc + pb[p]))) : 0.f; continue; }
            sc = (in && p < nh) ? sc : -INFINITY;
            const float mn = fmaxf(m[p], warp_max(sc));
            if (mn == -INFINITY) { pr[p] = 0.f; continue; }
            const float corr = expf(m[p] - mn);
            pr[p] = expf(sc - mn);
            l[p] = l[p] * corr + warp_sum(pr[p]);
            m[p] = mn;
#pragma unroll
            for (int v = 0; v < NV; ++v) acc[p][v] *= corr;
        }
        const int nvalid = min(KT, jmax - j0 + 1);
        const int dv0 = lane * NV;
        for (int jj0 = 0; jj0 < nvalid; jj0 += VR) {               // VR value rows in flight
            float vv[VR][NV];
#pragma unroll
            for (int u = 0; u < VR; ++u) {
                const long long voj = __shfl_sync(0xffffffffu, vo, (jj0 + u) & 31);
                if (jj0 + u < nvalid && dv0 < Dv) load_values<TC, NV>(vc + voj + dv0, vvec, Dv - dv0, vv[u]);
                else {
#pragma unroll
                    for (int v = 0; v < NV; ++v) vv[u][v] = 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < VR; ++u) {
#pragma unroll
                for (int p = 0; p < DPAIRS; ++p) {
                    const float pj = __shfl_sync(0xffffffffu, pr[p], (jj0 + u) & 31);
#pragma unroll
                    for (int v = 0; v < NV; ++v) acc[p][v] = fmaf(jj0 + u < nvalid ? pj : 0.f, vv[u][v], acc[p][v]);
                }
            }
        }
    }
    // fold the warps
#pragma unroll
    for (int p = 0; p < DPAIRS; ++p) {
        if (lane == 0) { st_m[warp * DPAIRS + p] = m[p]; st_l[warp * DPAIRS + p] = l[p]; }
#pragma unroll
        for (int v = 0; v < NV; ++v)
            if (lane * NV + v < Dv) st_acc[((size_t)warp * DPAIRS + p) * Dv + lane * NV + v] = acc[p][v];
    }
    __syncthreads();
    const size_t t = t0;
    for (int i = threadIdx.x; i < nh * Dv; i += blockDim.x) {
        const int p = i / Dv, dv = i - p * Dv;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARP; ++w) M = fmaxf(M, st_m[w * DPAIRS + p]);
        float L = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < NWARP; ++w) {
            const float mw = st_m[w * DPAIRS + p];
            if (mw != -INFINITY) {
                const float e = expf(mw - M);
                L = fmaf(st_l[w * DPAIRS + p], e, L);
                o = fmaf(st_acc[((size_t)w * DPAIRS + p) * Dv + dv], e, o);
            }
        }
        const int h = hb0 + p;
        if (a.splits > 1) {
            float* rec = a.ws + ((t * a.H + h) * a.splits + blockIdx.z) * (Dv + 2);
            if (dv == 0) { rec[0] = M; rec[1] = L; }
            rec[2 + dv] = o;
        } else {
            o = L > 0.f ? o / L : 0.f;
            if (a.gate) {
                const int u = (i - (int)threadIdx.x) >> 8;
                float z = 0.f;
#pragma unroll
                for (int uu = 0; uu < GPT; ++uu)
                    if (uu == u) z = gz[uu];
                if (u >= GPT) z = gate_logit(a, t, h, dv);
                o *= 1.f / (1.f + expf(-z));
            }
            a.out[t * a.ldo + (size_t)h * Dv + dv] = o * a.out_mult;
        }
    }
    if (a.splits == 1) return;
    __shared__ unsigned last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* tk = a.tickets + (size_t)blockIdx.x * gridDim.y + blockIdx.y;
        const unsigned n = atomicAdd(tk, 1u);
        last = (n == (unsigned)a.splits - 1u);
        if (last) *tk = 0u;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    __shared__ float wsl[DPAIRS][64];
    if (warp < nh) {                                   // weights of the slices: one warp per head, lanes over slices
        const float* rec = a.ws + ((t * a.H + hb0 + warp) * a.splits) * (Dv + 2);
        float ms[2], ls[2], M = -INFINITY;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int sp = lane + 32 * u;
            ms[u] = sp < a.splits ? __ldcg(rec + (size_t)sp * (Dv + 2)) : -INFINITY;
            ls[u] = sp < a.splits ? __ldcg(rec + (size_t)sp * (Dv + 2) + 1) : 0.f;
            M = fmaxf(M, ms[u]);
        }
        M = warp_max(M);
        float e[2], L = 0.f;
#pragma unroll
        for (int u = 0; u < 2; ++u) { e[u] = ms[u] == -INFINITY ? 0.f : expf(ms[u] - M); L += ls[u] * e[u]; }
        L = warp_sum(L);
        const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
        for (int u = 0; u < 2; ++u)
            if (lane + 32 * u < a.splits) wsl[warp][lane + 32 * u] = e[u] * inv;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nh * Dv; i += blockDim.x) {
        const int p = i / Dv, dv = i - p * Dv, h = hb0 + p;
        const float* rec = a.ws + ((t * a.H + h) * a.splits) * (Dv + 2) + 2 + dv;
        float o = 0.f;
#pragma unroll 8
        for (int sp = 0; sp < a.splits; ++sp) o = fmaf(wsl[p][sp], __ldcg(rec + (size_t)sp * (Dv + 2)), o);
        if (a.gate) {
            const int u = (i - (int)threadIdx.x) >> 8;
            float z = 0.f;
#pragma unroll
            for (int uu = 0; uu < GPT; ++uu)
                if (uu == u) z = gz[uu];
            if (u >= GPT) z = gate_logit(a, t, h, dv);
            o *= 1.f / (1.f + expf(-z));
        }
        a.out[t * a.ldo + (size_t)h * Dv + dv] = o * a.out_mult;
    }
}

template <typename TC, int NV, int DPAIRS>
int launch_attn_decode_dp(const AttnArgs& a, int tiles, cudaStream_t st) {
    const size_t smem = sizeof(float) * ((size_t)DPAIRS * a.D + 2 * NWARP * DPAIRS + (size_t)NWARP * DPAIRS * a.Dv);
    PGK_REQUIRE(smem <= 200 * 1024, "seq_attention failed: head sizes %d / %d need %zu bytes of shared memory", a.D, a.Dv, smem);
    static bool configured = false;
    if (smem > 32 * 1024 && !configured) {            // dynamic + static shared memory may pass 48 KB from here on
        PGK_CUDA(cudaFuncSetAttribute(seq_attention_decode_kernel<TC, NV, DPAIRS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = true;
    }
    const int rep = a.H / a.G, hsplit = (rep + DPAIRS - 1) / DPAIRS;
    PGK_CUDA(launch(seq_attention_decode_kernel<TC, NV, DPAIRS>, dim3(tiles, a.G * hsplit, a.splits), dim3(256), smem, st, a));
    return 0;
}

// Few blocks (one or a handful of requests): two heads per block instead of eight -- four times the blocks, a quarter of
// the instructions on each warp's critical path; the K/V rows are then read four times, from L2.
template <typename TC, int NV>
int launch_attn_decode(const AttnArgs& a, int tiles, cudaStream_t st) {
    const int rep = a.H / a.G;
    const long long blocks8 = (long long)tiles * a.G * ((rep + DPAIRS_MAX - 1) / DPAIRS_MAX) * a.splits;
    if (NV > 8 || (rep > 2 && blocks8 * 4 <= 2 * 148)) return launch_attn_decode_dp<TC, NV, 2>(a, tiles, st);
    if constexpr (NV <= 8) return launch_attn_decode_dp<TC, NV, DPAIRS_MAX>(a, tiles, st);
    return 1;
}

template <typename TC>
int launch_attn_decode_nv(const AttnArgs& a, int tiles, cudaStream_t st) {
    const int nv = (a.Dv + 31) / 32;
    if (nv <= 1) return launch_attn_decode<TC, 1>(a, tiles, st);
    if (nv <= 2) return launch_attn_decode<TC, 2>(a, tiles, st);
    if (nv <= 4) return launch_attn_decode<TC, 4>(a, tiles, st);
    if (nv <= 8) return launch_attn_decode<TC, 8>(a, tiles, st);
    if (nv <= 16) return launch_attn_decode<TC, 16>(a, tiles, st);
    set_error("seq_attention failed: value size %d exceeds 512", a.Dv);
    return 1;
}

}  // namespace

extern "C" {

int pgk_seq_heads_per_block(int heads, int kv_heads) {
    const int rep = kv_heads > 0 ? heads / kv_heads : 1;
    return rep < NWARP * PPW ? (rep > 0 ? rep : 1) : NWARP * PPW;
}
int pgk_seq_queries_per_tile(int heads, int kv_heads) { return (NWARP * PPW) / pgk_seq_heads_per_block(heads, kv_heads); }

int pgk_seq_mixer_prep(float* proj, int ld, int tokens, int heads, int kv_heads, int dim, int vdim, const float* q_weight,
                       const float* k_weight, float eps, int v_mode, float lam, float* v_first, void* k_cache, void* v_cache,
                       int cache_dtype, const int32_t* table, int max_pages, int page_size, const int32_t* slot,
                       const int32_t* pos, void* stream) {
    PGK_REQUIRE(cache_dtype == 0 || cache_dtype == 2, "seq_mixer_prep failed: the cache is float32 (0) or bfloat16 (2), got %d", cache_dtype);
    PGK_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0, "seq_mixer_prep failed: invalid head layout");
    PGK_REQUIRE(v_mode == 0 || v_first, "seq_mixer_prep failed: value mixing needs the v_first buffer");
    if (tokens <= 0) return 0;
    PrepArgs a{proj, ld, heads, kv_heads, dim, vdim, q_weight, k_weight, eps, v_mode, lam, v_first, k_cache, v_cache, table,
               max_pages, page_size, slot, pos};
    if (cache_dtype == 2) PGK_CUDA(launch(mixer_prep_kernel<uint16_t>, dim3(tokens, (heads + 2 * kv_heads + 3) / 4), dim3(128), 0, (cudaStream_t)stream, a));
    else PGK_CUDA(launch(mixer_prep_kernel<float>, dim3(tokens, (heads + 2 * kv_heads + 3) / 4), dim3(128), 0, (cudaStream_t)stream, a));
    return 0;
}

int pgk_seq_attention_ex(const float* q, int ldq, int q_off, const float* gate_rows, int ldg, int gate_off, int gate_mode,
                         float* out, int ldo, const void* k_cache, const void* v_cache, int k_ld, int v_ld, int cache_dtype,
                         const int32_t* table, int max_pages, int page_size, const int32_t* tiles, int n_tiles,
                         const float* slopes, const float* sinks, int heads, int kv_heads, int dim, int vdim, int chunk,
                         int window, float scale, float softcap, int splits, float* workspace, uint32_t* tickets,
                         int single_query, void* stream) {
    return pgk_seq_attention_ex2(q, ldq, q_off, gate_rows, ldg, gate_off, gate_mode, out, ldo, k_cache, v_cache, k_ld, v_ld,
                                 cache_dtype, table, max_pages, page_size, tiles, n_tiles, slopes, nullptr, sinks, heads,
                                 kv_heads, dim, vdim, chunk, window, 0, scale, softcap, 0, nullptr, 1.f, splits, workspace, tickets,
                                 single_query, stream);
}

int pgk_seq_attention_ex2(const float* q, int ldq, int q_off, const float* gate_rows, int ldg, int gate_off, int gate_mode,
                          float* out, int ldo, const void* k_cache, const void* v_cache, int k_ld, int v_ld, int cache_dtype,
                          const int32_t* table, int max_pages, int page_size, const int32_t* tiles, int n_tiles,
                          const float* slopes, const float* slopes2, const float* sinks, int heads, int kv_heads, int dim,
                          int vdim, int chunk, int window, int keep_first, float scale, float softcap, int weight_mode,
                          const float* weight_bias, float out_mult, int splits, float* workspace, uint32_t* tickets,
                          int single_query, void* stream) {
    PGK_REQUIRE(keep_first >= 0 && (keep_first == 0 || (window > 0 && chunk == 0)),
                "seq_attention failed: kept first positions need a window and no chunks");
    PGK_REQUIRE(!slopes2 || slopes, "seq_attention failed: the logarithmic distance term needs both per-head vectors");
    PGK_REQUIRE(weight_mode == 0 || (weight_mode == 1 && !sinks), "seq_attention failed: weight mode %d", weight_mode);
    PGK_REQUIRE(cache_dtype == 0 || cache_dtype == 2, "seq_attention failed: the cache is float32 (0) or bfloat16 (2), got %d", cache_dtype);
    PGK_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0, "seq_attention failed: invalid head layout");
    PGK_REQUIRE(splits >= 1 && splits <= 64 && (splits == 1 || (workspace && tickets)),
                "seq_attention failed: 1..64 key slices, more than one needs the workspace and the tickets");
    PGK_REQUIRE(gate_mode >= 0 && gate_mode <= 2 && (gate_mode == 0 || gate_rows), "seq_attention failed: gate mode %d", gate_mode);
    PGK_REQUIRE(k_ld >= dim && v_ld >= vdim && chunk >= 0 && window >= 0, "seq_attention failed: row strides %d / %d below the head sizes", k_ld, v_ld);
    if (n_tiles <= 0) return 0;
    AttnArgs a{};
    a.proj = q; a.ld = ldq; a.q_off = q_off; a.g_off = gate_off;
    a.out = out; a.ldo = ldo;
    a.kc = k_cache; a.vc = v_cache; a.table = table; a.max_pages = max_pages; a.PS = page_size;
    a.gsrc = gate_rows; a.ldg = ldg; a.sinks = sinks; a.window = window; a.kld = k_ld; a.vld = v_ld;
    a.valias = (k_cache == v_cache && k_ld == v_ld && vdim <= dim) ? 1 : 0;
    a.tiles = (const int4*)tiles; a.slopes = slopes; a.slopes2 = slopes2;
    a.keep = window > 0 ? keep_first : 0; a.prob = weight_mode; a.pbias = weight_bias; a.out_mult = out_mult;
    a.H = heads; a.G = kv_heads; a.D = dim; a.Dv = vdim; a.chunk = chunk;
    a.HB = pgk_seq_heads_per_block(heads, kv_heads); a.gate = gate_mode;
    a.scale = scale; a.cap = softcap; a.splits = splits; a.ws = workspace; a.tickets = tickets;
    if (single_query)       // every tile holds one query: the decoding kernel
        return cache_dtype == 2 ? launch_attn_decode_nv<uint16_t>(a, n_tiles, (cudaStream_t)stream)
                                : launch_attn_decode_nv<float>(a, n_tiles, (cudaStream_t)stream);
    return cache_dtype == 2 ? launch_attn_nv<uint16_t>(a, n_tiles, (cudaStream_t)stream)
                            : launch_attn_nv<float>(a, n_tiles, (cudaStream_t)stream);
}

int pgk_seq_attention(const float* proj, int ld, int q_off, int gate_off, float* out, int ldo, const void* k_cache,
                      const void* v_cache, int cache_dtype, const int32_t* table, int max_pages, int page_size,
                      const int32_t* tiles, int n_tiles, const float* slopes, int heads, int kv_heads, int dim, int vdim,
                      int chunk, float scale, float softcap, int gate, int splits, float* workspace, uint32_t* tickets,
                      int single_query, void* stream) {
    return pgk_seq_attention_ex(proj, ld, q_off, proj, ld, gate_off, gate ? 1 : 0, out, ldo, k_cache, v_cache, dim, vdim,
                                cache_dtype, table, max_pages, page_size, tiles, n_tiles, slopes, nullptr, heads, kv_heads,
                                dim, vdim, chunk, 0, scale, softcap, splits, workspace, tickets, single_query, stream);
}

// ---- whole-projection norm: q and k are normalised over ALL their heads at once; biases; values = keys before the norm
int pgk_seq_mixer_prep_all(float* proj, int ld, int tokens, int heads, int kv_heads, int dim, int k_off, const float* q_bias,
                           const float* k_bias, const float* q_weight, const float* k_weight, float weight_offset, float eps,
                           void* k_cache, void* v_cache, int cache_dtype, const int32_t* table, int max_pages, int page_size,
                           const int32_t* slot, const int32_t* pos, void* stream) {
    PGK_REQUIRE(cache_dtype == 0 || cache_dtype == 2, "seq_mixer_prep_all failed: the cache is float32 (0) or bfloat16 (2), got %d", cache_dtype);
    PGK_REQUIRE(heads > 0 && kv_heads > 0 && dim > 0, "seq_mixer_prep_all failed: invalid head layout");
    if (tokens <= 0) return 0;
    PrepAllArgs a{proj, ld, heads, kv_heads, dim, k_off, q_bias, k_bias, q_weight, k_weight, weight_offset, eps, k_cache, v_cache,
                  table, max_pages, page_size, slot, pos};
    if (cache_dtype == 2) PGK_CUDA(launch(mixer_prep_all_kernel<uint16_t>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, a));
    else PGK_CUDA(launch(mixer_prep_all_kernel<float>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, a));
    return 0;
}
int pgk_seq_decode_heads_per_block(void) { return DPAIRS_MAX; }

// ---- rotary positions (half layout) and a per-head norm with or without weights, K / V rows into the cache
int pgk_seq_mixer_prep_rot(float* proj, int ld, int tokens, int heads, int kv_heads, int dim, int vdim, int q_off, int k_off,
                           int v_off, int rot_dims, const double* inv_freq, int norm_mode, const float* q_weight,
                           const float* k_weight, float eps, void* k_cache, void* v_cache, int cache_dtype, const int32_t* table,
                           int max_pages, int page_size, const int32_t* slot, const int32_t* pos, void* stream) {
    return pgk_seq_mixer_prep_rot_ex(proj, ld, tokens, heads, kv_heads, dim, vdim, q_off, k_off, v_off, rot_dims, inv_freq, norm_mode,
                                     q_weight, k_weight, eps, nullptr, nullptr, nullptr, nullptr, k_cache, v_cache, cache_dtype, table,
                                     max_pages, page_size, slot, pos, stream);
}

// ---- the same with projection biases on q, k and v and a factor on every query head
int pgk_seq_mixer_prep_rot_ex(float* proj, int ld, int tokens, int heads, int kv_heads, int dim, int vdim, int q_off, int k_off,
                              int v_off, int rot_dims, const double* inv_freq, int norm_mode, const float* q_weight,
                              const float* k_weight, float eps, const float* q_bias, const float* k_bias, const float* v_bias,
                              const float* q_mult, void* k_cache, void* v_cache, int cache_dtype, const int32_t* table,
                              int max_pages, int page_size, const int32_t* slot, const int32_t* pos, void* stream) {
    PGK_REQUIRE(cache_dtype == 0 || cache_dtype == 2, "seq_mixer_prep_rot failed: the cache is float32 (0) or bfloat16 (2), got %d", cache_dtype);
    PGK_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0, "seq_mixer_prep_rot failed: invalid head layout");
    PGK_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim && (rot_dims == 0 || inv_freq),
                "seq_mixer_prep_rot failed: %d rotated dimensions in heads of %d", rot_dims, dim);
    PGK_REQUIRE(norm_mode >= 0 && norm_mode <= 2 && (norm_mode != 2 || (q_weight && k_weight)), "seq_mixer_prep_rot failed: norm mode %d", norm_mode);
    if (tokens <= 0) return 0;
    PrepRotArgs a{proj, ld, heads, kv_heads, dim, vdim, q_off, k_off, v_off, rot_dims, inv_freq, norm_mode, q_weight, k_weight, eps,
                  k_cache, v_cache, table, max_pages, page_size, slot, pos, q_bias, k_bias, v_bias, q_mult};
    const dim3 grid(tokens, (heads + 2 * kv_heads + 3) / 4);
    if (cache_dtype == 2) PGK_CUDA(launch(mixer_prep_rot_kernel<uint16_t>, grid, dim3(128), 0, (cudaStream_t)stream, a));
    else PGK_CUDA(launch(mixer_prep_rot_kernel<float>, grid, dim3(128), 0, (cudaStream_t)stream, a));
    return 0;
}

}  // extern "C"
