// seq_gated.cu -- the token-major models' pieces with DATA-DEPENDENT gates, all in float32:
//
//   dyt_rows           tanh(alpha x) * w + b on rows (a pointwise squashing in the place of a norm: no statistic of the row); rows may be gathered, and the
//                      result may be added to the output (a normalised branch joining the residual stream)
//   rms_pair_rows      mult * (a / rms(a) * wa + b / rms(b) * wb): two branches joined after an RMS norm each
//   polynorm_rows      c0 z / rms(z) + c1 z^2 / rms(z^2) + c2 z^3 / rms(z^3) + c3, in place on the rows of a feed-forward
//   moe_route_biased   softmax over all router outputs; the `top` largest of score + bias are chosen, their weights are the
//                      scores themselves (renormalised on request); router outputs >= real_experts stand for experts without
//                      matrices (`mat` = -1 for them)
//   moe_combine_rows   out = sum_k w[t, k] * (parts row, or the token's own input row for an expert without matrices)
//                      + sigmoid(gate logit) * shared expert row
//   dyt_seam           a sublayer's result (plain rows, the two-branch join, or the expert sum) through the norm behind it into
//                      the residual stream, and the next sublayer's norm of the sum, in one launch
//   gated_prep         q <- silu(q), f <- low + (1 - low) sigmoid(f + bias) on the fused projection row
//   delta_prep         q, k heads to unit length (q also times dim^-1/2); beta <- sigmoid(beta); g <- exp(-exp(A_log)
//                      softplus(a + dt_bias))
//   gated_recurrence   the state S [dim][vdim] of every (sequence, head) walked token by token:
//                        gated outer product:  S <- diag(a_t) S + k_t v_t^T,  o_t = S^T q_t     (k_t = 1 - a_t when no keys)
//                        delta rule:           S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//                      A block owns 2 value columns per warp; the rows of S are dealt to the sixteen lanes of a column in groups of
//                      four, each lane keeps its share in registers, the step's q / k / a rows arrive in shared memory 16 tokens
//                      at a time by asynchronous copies, the next chunk while this one is walked.  One decoded token is a walk of one.  A sequence whose first position is 0 starts from
//                      zero, whatever its slot held.
#include "common.cuh"
#include "../../include/pgk_b200.h"

using namespace pgk;

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nw; ++i) s += red[i];
    return s;
}

// ---------------------------------------------------------------- dynamic tanh
__global__ void __launch_bounds__(256) dyt_rows_kernel(const float* x, const int* src_rows, float alpha, const float* w,
                                                       const float* b, float* out, int W, int accumulate) {
    const int t = blockIdx.x;
    const size_t srow = src_rows ? (size_t)src_rows[t] : (size_t)t;
    for (int i = blockIdx.y * 256 + threadIdx.x; i < W; i += gridDim.y * 256) {
        const float r = fmaf(tanhf(alpha * x[srow * W + i]), w[i], b ? b[i] : 0.f);
        float* o = out + (size_t)t * W + i;
        *o = accumulate ? *o + r : r;
    }
}

// ---------------------------------------------------------------- two branches, an RMS norm each
__global__ void __launch_bounds__(256) rms_pair_rows_kernel(const float* a, const float* wa, const float* b, const float* wb,
                                                            float eps, float mult, float* out, int W) {
    __shared__ float red[8];
    const size_t o = (size_t)blockIdx.x * W;
    float qa = 0.f, qb = 0.f;
    for (int i = threadIdx.x; i < W; i += 256) {
        const float u = a[o + i], v = b[o + i];
        qa = fmaf(u, u, qa);
        qb = fmaf(v, v, qb);
    }
    const float ia = 1.f / sqrtf(block_sum(qa, red) / (float)W + eps);
    const float ib = 1.f / sqrtf(block_sum(qb, red) / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += 256) out[o + i] = mult * (a[o + i] * ia * wa[i] + b[o + i] * ib * wb[i]);
}

// ---------------------------------------------------------------- polynomial activation with an RMS norm per power
__global__ void __launch_bounds__(256) polynorm_rows_kernel(float* z, int ld, const float* coef, float eps, int n) {
    __shared__ float red[8];
    float* row = z + (size_t)blockIdx.x * ld;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) {
        const float v = row[i], v2 = v * v, v3 = v2 * v;
        s1 = fmaf(v, v, s1);
        s2 = fmaf(v2, v2, s2);
        s3 = fmaf(v3, v3, s3);
    }
    const float i1 = coef[0] / sqrtf(block_sum(s1, red) / (float)n + eps);
    const float i2 = coef[1] / sqrtf(block_sum(s2, red) / (float)n + eps);
    const float i3 = coef[2] / sqrtf(block_sum(s3, red) / (float)n + eps);
    const float c3 = coef[3];
    for (int i = threadIdx.x; i < n; i += 256) {
        const float v = row[i], v2 = v * v;
        row[i] = fmaf(v, i1, fmaf(v2, i2, fmaf(v2 * v, i3, c3)));
    }
}

// ---------------------------------------------------------------- router with a choice bias
struct RouteBiasArgs {
    const float* z; int ldz, T, E, real, top, renorm;
    const float* bias;
    int* idx; int* mat; float* wt; int* rank; int* counts;
};

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

constexpr int ROUTE_WARPS = 4;       // tokens per block, a warp each

__global__ void __launch_bounds__(ROUTE_WARPS * 32) moe_route_biased_kernel(RouteBiasArgs a) {
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= a.T) return;
    float* s = sm + (size_t)warp * 2 * a.E;       // [E] scores
    float* c = s + a.E;                           // [E] choice scores; -inf once chosen
    const float* z = a.z + (size_t)t * a.ldz;
    float mx = -INFINITY;
    for (int e = lane; e < a.E; e += 32) { const float v = z[e]; s[e] = v; mx = fmaxf(mx, v); }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < a.E; e += 32) { const float p = expf(s[e] - mx); s[e] = p; sum += p; }
    sum = warp_sum(sum);
    for (int e = lane; e < a.E; e += 32) { s[e] = s[e] / sum; c[e] = s[e] + (a.bias ? a.bias[e] : 0.f); }
    __syncwarp();
    float wsum = 0.f;
    for (int k = 0; k < a.top; ++k) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < a.E; e += 32)
            if (c[e] > bv) { bv = c[e]; bi = e; }
        warp_argmax(bv, bi);
        __syncwarp();
        if (lane == 0) {
            c[bi] = -INFINITY;
            const size_t o = (size_t)t * a.top + k;
            a.idx[o] = bi;
            a.mat[o] = bi < a.real ? bi : -1;
            a.wt[o] = s[bi];
            if (a.counts) a.rank[o] = atomicAdd(&a.counts[bi], 1);
        }
        wsum += s[bi];
        __syncwarp();
    }
    if (a.renorm) {
        __syncwarp();
        for (int k = lane; k < a.top; k += 32) a.wt[(size_t)t * a.top + k] /= (wsum + 1e-20f);
    }
}

// ---------------------------------------------------------------- weighted sum of the chosen experts + gated shared expert
struct CombineArgs {
    const float* parts; const int* inv; const int* mat; const float* w; int top;
    const float* self_rows;                         // the token's own input rows: the output of an expert without matrices
    const float* shared; const float* gate; int ldg, gate_off;     // shared expert rows times sigmoid(gate[t, gate_off])
    float* out; int W;
};

constexpr int CTOP = 64;

// the (token, slot) rows of token t staged for the whole block: weights and row offsets in parts (-1: the token's own row)
__device__ __forceinline__ void combine_stage(const CombineArgs& a, int t, float* wk, long long* pk) {
    if (threadIdx.x < a.top && threadIdx.x < CTOP) {
        const size_t o = (size_t)t * a.top + threadIdx.x;
        wk[threadIdx.x] = a.w[o];
        pk[threadIdx.x] = (a.mat && a.mat[o] < 0) ? -1 : (long long)a.inv[o] * a.W;
    }
    __syncthreads();
}

__device__ __forceinline__ float combine_value(const CombineArgs& a, int t, int i, const float* wk, const long long* pk, float sg) {
    float v = 0.f;
    const int top = a.top, ks = top < CTOP ? top : CTOP;
    for (int k = 0; k < ks; ++k)
        v = fmaf(wk[k], pk[k] < 0 ? a.self_rows[(size_t)t * a.W + i] : a.parts[pk[k] + i], v);
    for (int k = CTOP; k < top; ++k) {
        const size_t o = (size_t)t * top + k;
        const bool self = a.mat && a.mat[o] < 0;
        v = fmaf(a.w[o], self ? a.self_rows[(size_t)t * a.W + i] : a.parts[(size_t)a.inv[o] * a.W + i], v);
    }
    if (a.shared) v = fmaf(sg, a.shared[(size_t)t * a.W + i], v);
    return v;
}

__device__ __forceinline__ float combine_gate(const CombineArgs& a, int t) {
    return a.shared ? (a.gate ? sigmoid_f(a.gate[(size_t)t * a.ldg + a.gate_off]) : 1.f) : 0.f;
}

__global__ void __launch_bounds__(256) moe_combine_rows_kernel(CombineArgs a) {
    __shared__ float wk[CTOP];
    __shared__ long long pk[CTOP];
    const int t = blockIdx.x;
    combine_stage(a, t, wk, pk);
    const float sg = combine_gate(a, t);
    for (int i = threadIdx.x; i < a.W; i += 256) a.out[(size_t)t * a.W + i] = combine_value(a, t, i, wk, pk, sg);
}

// ---------------------------------------------------------------- a sublayer's result joins the residual stream
// One launch for the seam behind a sublayer of a block with norms on both sides: the sublayer's result v -- plain rows
// (mode 0), two branches after an RMS norm each (mode 1), or the weighted sum of expert rows with the gated shared expert
// (mode 2) -- passes the norm behind the sublayer and joins the residual stream, x += tanh(alpha1 v) w1 + b1, and the norm in
// front of the next sublayer is taken from the sum at once, h = tanh(alpha2 x) w2 + b2 (h NULL: not wanted).
struct SeamArgs {
    int mode;
    const float* y; const float* y2; const float* wa; const float* wb; float mult, eps;
    CombineArgs c;
    float alpha1; const float* w1; const float* b1;
    float* x;
    float alpha2; const float* w2; const float* b2; float* h;
    int W;
};

__global__ void __launch_bounds__(256) dyt_seam_kernel(SeamArgs a) {
    __shared__ float red[8];
    __shared__ float wk[CTOP];
    __shared__ long long pk[CTOP];
    const int t = blockIdx.x, W = a.W;
    const size_t o = (size_t)t * W;
    float ia = 0.f, ib = 0.f, sg = 0.f;
    if (a.mode == 1) {
        float qa = 0.f, qb = 0.f;
        for (int i = threadIdx.x; i < W; i += 256) {
            const float u = a.y[o + i], v = a.y2[o + i];
            qa = fmaf(u, u, qa);
            qb = fmaf(v, v, qb);
        }
        ia = a.mult / sqrtf(block_sum(qa, red) / (float)W + a.eps);
        ib = a.mult / sqrtf(block_sum(qb, red) / (float)W + a.eps);
    } else if (a.mode == 2) {
        combine_stage(a.c, t, wk, pk);
        sg = combine_gate(a.c, t);
    }
    // few rows: gridDim.y blocks share a row's columns (each forms the row's two sums itself in mode 1)
    for (int i = blockIdx.y * 256 + threadIdx.x; i < W; i += gridDim.y * 256) {
        float v;
        if (a.mode == 0) v = a.y[o + i];
        else if (a.mode == 1) v = a.y[o + i] * ia * a.wa[i] + a.y2[o + i] * ib * a.wb[i];
        else v = combine_value(a.c, t, i, wk, pk, sg);
        const float xv = a.x[o + i] + fmaf(tanhf(a.alpha1 * v), a.w1[i], a.b1 ? a.b1[i] : 0.f);
        a.x[o + i] = xv;
        if (a.h) a.h[o + i] = fmaf(tanhf(a.alpha2 * xv), a.w2[i], a.b2 ? a.b2[i] : 0.f);
    }
}

// ---------------------------------------------------------------- preparation of the gated outer-product recurrence
// units per token: H query heads (silu), H gate heads (f <- low + (1 - low) sigmoid(f + bias)); a warp each
__global__ void __launch_bounds__(128) gated_prep_kernel(float* proj, int ld, int H, int D, int q_off, int f_off,
                                                         const float* f_bias, const float* low) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, u = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (u >= 2 * H) return;
    float* row = proj + (size_t)t * ld;
    if (u < H) {
        float* q = row + q_off + (size_t)u * D;
        for (int d = lane; d < D; d += 32) q[d] = silu_f(q[d]);
        return;
    }
    const int h = u - H;
    float* f = row + f_off + (size_t)h * D;
    for (int d = lane; d < D; d += 32) {
        const float lo = low ? low[h * D + d] : 0.f;
        f[d] = lo + (1.f - lo) * sigmoid_f(f[d] + (f_bias ? f_bias[h * D + d] : 0.f));
    }
}

// ---------------------------------------------------------------- preparation of the delta rule
// units per token: G query heads, G key heads (unit length; q also times dim^-1/2), then one more unit for the H (beta, g) pairs
struct DeltaPrepArgs {
    float* qk; int ldqk, q_off, k_off;              // rows that hold the q and k heads after their convolution
    float* proj; int ld, b_off, a_off;              // rows that hold beta and a as projected
    const float* A_log; const float* dt_bias;
    int H, G, D; float q_mult;
};

__global__ void __launch_bounds__(128) delta_prep_kernel(DeltaPrepArgs a) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, u = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (u > 2 * a.G) return;
    if (u == 2 * a.G) {
        float* row = a.proj + (size_t)t * a.ld;
        for (int h = lane; h < a.H; h += 32) {
            row[a.b_off + h] = sigmoid_f(row[a.b_off + h]);
            row[a.a_off + h] = expf(-expf(a.A_log[h]) * softplus_f(row[a.a_off + h] + a.dt_bias[h]));
        }
        return;
    }
    const bool is_k = u >= a.G;
    float* x = a.qk + (size_t)t * a.ldqk + (is_k ? a.k_off + (size_t)(u - a.G) * a.D : a.q_off + (size_t)u * a.D);
    float ss = 0.f;
    for (int d = lane; d < a.D; d += 32) ss = fmaf(x[d], x[d], ss);
    const float inv = (is_k ? 1.f : a.q_mult) / sqrtf(warp_sum(ss) + 1e-6f);
    for (int d = lane; d < a.D; d += 32) x[d] *= inv;
}

// ---------------------------------------------------------------- the recurrence
constexpr int GR = 16;                // lanes per value column
constexpr int GCW = 32 / GR;          // value columns per warp
constexpr int GWARPS = 8;             // warps per block
constexpr int GCOLS = GWARPS * GCW;   // value columns per block
constexpr int GTC = 16;               // tokens per staged chunk
constexpr int GTHREADS = GWARPS * 32;

struct GatedArgs {
    const float* q; int ldq, q_off;   // head hq at q_off + hq * D of row t; hq = h / (H / G)
    const float* k; int ldk, k_off;   // may be NULL in the gated outer-product form: k = 1 - a
    const float* a; int lda, a_off;   // gated outer product: decays [G heads x D]; delta rule: g, one per value head
    const float* b; int ldb, b_off;   // delta rule: beta, one per value head
    const float* v; int ldv, v_off;   // value head h at v_off + h * Dv
    float* out; int ldo;              // out[t, h * Dv + c]
    float* state;                     // [slots][H][D][Dv]
    const int4* seqs;                 // (first row, rows, slot, first position)
    int H, G, D, Dv;
    int vec;                          // every row, offset and size a multiple of 16 bytes: chunks arrive by asynchronous copies
};

__device__ __forceinline__ void cp_async16(void* smem, const void* g) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* g) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem)), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One stage of the chunk pipeline in shared memory: Q [GTC][Dp], K [GTC][Dp], then the decays [GTC][Dp] (gated outer product)
// or g, beta and q.k per token [3][GTC] (delta rule), then V [GTC][GCOLS].  Dp = D rounded up to 4 GR; rows D .. Dp - 1 and value
// columns beyond Dv are zeroed once and never written again.
template <bool DELTA> __device__ __forceinline__ int stage_floats(int Dp) {
    return 2 * GTC * Dp + (DELTA ? 3 * GTC : GTC * Dp) + GTC * GCOLS;
}

// the chunk of nc tokens from row r0 on, by 16-byte asynchronous copies (the caller commits the group)
template <bool DELTA>
__device__ __forceinline__ void stage_async(const GatedArgs& a, float* st, int Dp, int r0, int nc, int h, int hq, int col0) {
    const int D = a.D, D4 = D >> 2, tid = threadIdx.x;
    float* Qs = st;
    float* Ks = Qs + GTC * Dp;
    float* As = Ks + GTC * Dp;
    float* Vs = As + (DELTA ? 3 * GTC : GTC * Dp);
    for (int i = tid; i < nc * D4; i += GTHREADS) {
        const int t = i / D4, d = (i - t * D4) * 4;
        const size_t row = (size_t)(r0 + t);
        cp_async16(Qs + t * Dp + d, a.q + row * a.ldq + a.q_off + (size_t)hq * D + d);
        if (DELTA || a.k) cp_async16(Ks + t * Dp + d, a.k + row * a.ldk + a.k_off + (size_t)hq * D + d);
        if (!DELTA) cp_async16(As + t * Dp + d, a.a + row * a.lda + a.a_off + (size_t)hq * D + d);
    }
    for (int i = tid; i < nc * (GCOLS / 4); i += GTHREADS) {
        const int t = i / (GCOLS / 4), j = (i - t * (GCOLS / 4)) * 4;
        if (col0 + j < a.Dv) cp_async16(Vs + t * GCOLS + j, a.v + (size_t)(r0 + t) * a.ldv + a.v_off + (size_t)h * a.Dv + col0 + j);
    }
    if (DELTA && tid < nc) {
        const size_t row = (size_t)(r0 + tid);
        cp_async4(As + tid, a.a + row * a.lda + a.a_off + h);
        cp_async4(As + GTC + tid, a.b + row * a.ldb + a.b_off + h);
    }
}

// the same chunk by plain loads (rows that are not 16-byte aligned)
template <bool DELTA>
__device__ __forceinline__ void stage_plain(const GatedArgs& a, float* st, int Dp, int r0, int nc, int h, int hq, int col0) {
    const int D = a.D, tid = threadIdx.x;
    float* Qs = st;
    float* Ks = Qs + GTC * Dp;
    float* As = Ks + GTC * Dp;
    float* Vs = As + (DELTA ? 3 * GTC : GTC * Dp);
    for (int i = tid; i < nc * D; i += GTHREADS) {
        const int t = i / D, d = i - t * D;
        const size_t row = (size_t)(r0 + t);
        Qs[t * Dp + d] = a.q[row * a.ldq + a.q_off + (size_t)hq * D + d];
        if (DELTA || a.k) Ks[t * Dp + d] = a.k[row * a.ldk + a.k_off + (size_t)hq * D + d];
        if (!DELTA) As[t * Dp + d] = a.a[row * a.lda + a.a_off + (size_t)hq * D + d];
    }
    for (int i = tid; i < nc * GCOLS; i += GTHREADS) {
        const int t = i / GCOLS, j = i - t * GCOLS;
        if (col0 + j < a.Dv) Vs[i] = a.v[(size_t)(r0 + t) * a.ldv + a.v_off + (size_t)h * a.Dv + col0 + j];
    }
    if (DELTA && tid < nc) {
        const size_t row = (size_t)(r0 + tid);
        As[tid] = a.a[row * a.lda + a.a_off + h];
        As[GTC + tid] = a.b[row * a.ldb + a.b_off + h];
    }
}

// NR: state rows per lane (a multiple of 4); rows 4 GR j + 4 r + e, j < NR / 4, e < 4 belong to lane group r
template <int NR, bool DELTA>
__global__ void __launch_bounds__(GTHREADS) gated_recurrence_kernel(GatedArgs a) {
    extern __shared__ __align__(16) float sm[];
    constexpr int RS = 4 * GR;                   // rows between a lane's groups of four
    const int D = a.D, Dp = (D + RS - 1) / RS * RS, nj = Dp / RS, SF = stage_floats<DELTA>(Dp);
    float* Os = sm + 2 * SF;                     // [GTC][GCOLS]
    const int4 sq = a.seqs[blockIdx.x];
    const int row0 = sq.x, n = sq.y, slot = sq.z, pos0 = sq.w;
    const int h = blockIdx.y, hq = h / (a.H / a.G), col0 = blockIdx.z * GCOLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane / GCW, cc = warp * GCW + (lane % GCW), c = col0 + cc;
    const bool live = c < a.Dv, keys = DELTA || a.k != nullptr;
    for (int i = tid; i < 2 * SF; i += GTHREADS) sm[i] = 0.f;
    float* Sg = a.state + (((size_t)slot * a.H + h) * D) * a.Dv + c;
    float S[NR];
#pragma unroll
    for (int j = 0; j < NR / 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int d = RS * j + 4 * r + e;
            S[4 * j + e] = (pos0 > 0 && live && d < D) ? Sg[(size_t)d * a.Dv] : 0.f;
        }
    __syncthreads();
    const int nchunks = (n + GTC - 1) / GTC;
    if (a.vec) {
        stage_async<DELTA>(a, sm, Dp, row0, min(GTC, n), h, hq, col0);
        cp_async_commit();
    }
    for (int ci = 0; ci < nchunks; ++ci) {
        float* st = sm + (ci & 1) * SF;
        const int c0 = ci * GTC, nc = min(GTC, n - c0);
        if (a.vec) {
            if (ci + 1 < nchunks) {              // the next chunk travels while this one is walked
                stage_async<DELTA>(a, sm + ((ci + 1) & 1) * SF, Dp, row0 + c0 + GTC, min(GTC, n - c0 - GTC), h, hq, col0);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
        } else {
            stage_plain<DELTA>(a, st, Dp, row0 + c0, nc, h, hq, col0);
        }
        __syncthreads();
        const float* Qs = st;
        const float* Ks = Qs + GTC * Dp;
        float* As = st + 2 * GTC * Dp;
        const float* Vs = As + (DELTA ? 3 * GTC : GTC * Dp);
        if (DELTA) {
            for (int t = warp; t < nc; t += GWARPS) {
                float s = 0.f;
                for (int d = lane; d < Dp; d += 32) s = fmaf(Qs[t * Dp + d], Ks[t * Dp + d], s);
                s = warp_sum(s);
                if (lane == 0) As[2 * GTC + t] = s;
            }
            __syncthreads();
        }
#pragma unroll 2
        for (int t = 0; t < nc; ++t) {
            const float* qr = Qs + t * Dp + 4 * r;
            const float* kr = Ks + t * Dp + 4 * r;
            const float vc = Vs[t * GCOLS + cc];
            if (DELTA) {
                float ks0 = 0.f, ks1 = 0.f, qs0 = 0.f, qs1 = 0.f;
#pragma unroll
                for (int j = 0; j < NR / 4; ++j) {
                    if (j < nj) {
                        const float4 q4 = *(const float4*)(qr + RS * j), k4 = *(const float4*)(kr + RS * j);
                        ks0 = fmaf(k4.x, S[4 * j], ks0); ks1 = fmaf(k4.y, S[4 * j + 1], ks1);
                        ks0 = fmaf(k4.z, S[4 * j + 2], ks0); ks1 = fmaf(k4.w, S[4 * j + 3], ks1);
                        qs0 = fmaf(q4.x, S[4 * j], qs0); qs1 = fmaf(q4.y, S[4 * j + 1], qs1);
                        qs0 = fmaf(q4.z, S[4 * j + 2], qs0); qs1 = fmaf(q4.w, S[4 * j + 3], qs1);
                    }
                }
                float ks = ks0 + ks1, qs = qs0 + qs1;
#pragma unroll
                for (int o = GCW; o < 32; o <<= 1) {
                    ks += __shfl_xor_sync(0xffffffffu, ks, o);
                    qs += __shfl_xor_sync(0xffffffffu, qs, o);
                }
                const float g = As[t], beta = As[GTC + t], qk = As[2 * GTC + t];
                const float u = beta * (vc - g * ks);
                if (r == 0) Os[t * GCOLS + cc] = fmaf(g, qs, qk * u);
#pragma unroll
                for (int j = 0; j < NR / 4; ++j) {
                    if (j < nj) {
                        const float4 k4 = *(const float4*)(kr + RS * j);
                        S[4 * j] = fmaf(g, S[4 * j], k4.x * u);
                        S[4 * j + 1] = fmaf(g, S[4 * j + 1], k4.y * u);
                        S[4 * j + 2] = fmaf(g, S[4 * j + 2], k4.z * u);
                        S[4 * j + 3] = fmaf(g, S[4 * j + 3], k4.w * u);
                    }
                }
            } else {
                const float* ar = As + t * Dp + 4 * r;
                float o0 = 0.f, o1 = 0.f;
#pragma unroll
                for (int j = 0; j < NR / 4; ++j) {
                    if (j < nj) {
                        const float4 q4 = *(const float4*)(qr + RS * j), a4 = *(const float4*)(ar + RS * j);
                        float4 k4;
                        if (keys) k4 = *(const float4*)(kr + RS * j);
                        else k4 = make_float4(1.f - a4.x, 1.f - a4.y, 1.f - a4.z, 1.f - a4.w);
                        S[4 * j] = fmaf(a4.x, S[4 * j], k4.x * vc);
                        S[4 * j + 1] = fmaf(a4.y, S[4 * j + 1], k4.y * vc);
                        S[4 * j + 2] = fmaf(a4.z, S[4 * j + 2], k4.z * vc);
                        S[4 * j + 3] = fmaf(a4.w, S[4 * j + 3], k4.w * vc);
                        o0 = fmaf(q4.x, S[4 * j], o0); o1 = fmaf(q4.y, S[4 * j + 1], o1);
                        o0 = fmaf(q4.z, S[4 * j + 2], o0); o1 = fmaf(q4.w, S[4 * j + 3], o1);
                    }
                }
                float o = o0 + o1;
#pragma unroll
                for (int sh = GCW; sh < 32; sh <<= 1) o += __shfl_xor_sync(0xffffffffu, o, sh);
                if (r == 0) Os[t * GCOLS + cc] = o;
            }
        }
        __syncthreads();
        for (int i = tid; i < nc * GCOLS; i += GTHREADS) {
            const int t = i / GCOLS, j = i - t * GCOLS;
            if (col0 + j < a.Dv) a.out[(size_t)(row0 + c0 + t) * a.ldo + (size_t)h * a.Dv + col0 + j] = Os[i];
        }
    }
    if (live) {
#pragma unroll
        for (int j = 0; j < NR / 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int d = RS * j + 4 * r + e;
                if (d < D) Sg[(size_t)d * a.Dv] = S[4 * j + e];
            }
    }
}

template <int NR, bool DELTA>
int launch_gated(const GatedArgs& a, int n_seqs, size_t smem, cudaStream_t st) {
    static bool configured = false;
    if (smem > 40 * 1024 && !configured) {
        PGK_CUDA(cudaFuncSetAttribute(gated_recurrence_kernel<NR, DELTA>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        configured = true;
    }
    PGK_CUDA(launch(gated_recurrence_kernel<NR, DELTA>, dim3(n_seqs, a.H, (a.Dv + GCOLS - 1) / GCOLS), dim3(GTHREADS), smem, st, a));
    return 0;
}

inline bool mult4(long long v) { return (v & 3) == 0; }
inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

template <bool DELTA>
int run_gated(GatedArgs a, int n_seqs, cudaStream_t st) {
    const int Dp = (a.D + 4 * GR - 1) / (4 * GR) * (4 * GR);
    const size_t smem = sizeof(float) * (2 * ((size_t)2 * GTC * Dp + (DELTA ? 3 * GTC : (size_t)GTC * Dp) + GTC * GCOLS) + GTC * GCOLS);
    a.vec = mult4(a.D) && mult4(a.Dv) && mult4(a.ldq) && mult4(a.q_off) && aligned16(a.q) && mult4(a.ldv) && mult4(a.v_off) &&
            aligned16(a.v) && (!a.k || (mult4(a.ldk) && mult4(a.k_off) && aligned16(a.k))) &&
            (DELTA || (mult4(a.lda) && mult4(a.a_off) && aligned16(a.a)));
    if (Dp <= 64) return launch_gated<64 / GR, DELTA>(a, n_seqs, smem, st);
    if (Dp <= 128) return launch_gated<128 / GR, DELTA>(a, n_seqs, smem, st);
    return launch_gated<256 / GR, DELTA>(a, n_seqs, smem, st);
}

}  // namespace

extern "C" {

int pgk_dyt_rows_f32(const float* x, const int32_t* src_rows, float alpha, const float* weight, const float* bias, float* out,
                     int rows, int width, int accumulate, void* stream) {
    PGK_REQUIRE(width > 0 && weight, "dyt_rows_f32 failed: width %d", width);
    if (rows <= 0) return 0;
    const int by = width > 4096 ? 4 : 1;
    PGK_CUDA(launch(dyt_rows_kernel, dim3(rows, by), dim3(256), 0, (cudaStream_t)stream, x, src_rows, alpha, weight, bias, out, width,
                    accumulate));
    return 0;
}

int pgk_rms_pair_rows_f32(const float* a, const float* weight_a, const float* b, const float* weight_b, float eps, float mult,
                          float* out, int rows, int width, void* stream) {
    PGK_REQUIRE(width > 0 && weight_a && weight_b, "rms_pair_rows_f32 failed: width %d", width);
    if (rows <= 0) return 0;
    PGK_CUDA(launch(rms_pair_rows_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, a, weight_a, b, weight_b, eps, mult, out, width));
    return 0;
}

int pgk_polynorm_rows_f32(float* z, int ld, const float* coef, float eps, int rows, int n, void* stream) {
    PGK_REQUIRE(n > 0 && ld >= n && coef, "polynorm_rows_f32 failed: %d columns in rows of %d", n, ld);
    if (rows <= 0) return 0;
    PGK_CUDA(launch(polynorm_rows_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, z, ld, coef, eps, n));
    return 0;
}

int pgk_moe_route_biased(const float* logits, int ld, int tokens, int outputs, int real_experts, int top, const float* bias,
                         int renorm, int32_t* idx, int32_t* mat, float* weights, int32_t* rank, int32_t* counts, void* stream) {
    PGK_REQUIRE(outputs > 0 && top > 0 && top <= outputs && real_experts >= 0 && real_experts <= outputs,
                "moe_route_biased failed: top %d of %d router outputs (%d with matrices)", top, outputs, real_experts);
    PGK_REQUIRE((rank == nullptr) == (counts == nullptr), "moe_route_biased failed: ranks and counts come together");
    if (tokens <= 0) return 0;
    RouteBiasArgs a{logits, ld, tokens, outputs, real_experts, top, renorm ? 1 : 0, bias, idx, mat, weights, rank, counts};
    const size_t smem = (size_t)ROUTE_WARPS * 2 * outputs * 4;
    PGK_REQUIRE(smem <= 48 * 1024, "moe_route_biased failed: too many router outputs (%d)", outputs);
    PGK_CUDA(launch(moe_route_biased_kernel, dim3((tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem,
                    (cudaStream_t)stream, a));
    return 0;
}

int pgk_moe_combine_rows_f32(const float* parts, const int32_t* inv, const int32_t* mat, const float* weights, int top,
                             const float* self_rows, const float* shared_rows, const float* gate_rows, int ldg, int gate_off,
                             float* out, int rows, int width, void* stream) {
    PGK_REQUIRE(width > 0 && top >= 0 && (top == 0 || (parts && inv && weights)), "moe_combine_rows_f32 failed: invalid arguments");
    PGK_REQUIRE(!mat || self_rows, "moe_combine_rows_f32 failed: experts without matrices need the tokens' own rows");
    if (rows <= 0) return 0;
    CombineArgs a{parts, inv, mat, weights, top, self_rows, shared_rows, gate_rows, ldg, gate_off, out, width};
    PGK_CUDA(launch(moe_combine_rows_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, a));
    return 0;
}

int pgk_dyt_seam_f32(int mode, const float* y, const float* y2, const float* weight_a, const float* weight_b, float mult, float eps,
                     const float* parts, const int32_t* inv, const int32_t* mat, const float* weights, int top,
                     const float* self_rows, const float* shared_rows, const float* gate_rows, int ldg, int gate_off,
                     float alpha1, const float* w1, const float* b1, float* x, float alpha2, const float* w2, const float* b2,
                     float* h, int rows, int width, void* stream) {
    PGK_REQUIRE(mode >= 0 && mode <= 2 && width > 0 && w1 && x && (!h || w2), "dyt_seam_f32 failed: mode %d, width %d", mode, width);
    PGK_REQUIRE(mode == 2 || y, "dyt_seam_f32 failed: the sublayer's rows are missing");
    PGK_REQUIRE(mode != 1 || (y2 && weight_a && weight_b), "dyt_seam_f32 failed: two branches need both rows and both weight vectors");
    PGK_REQUIRE(mode != 2 || (top >= 0 && (top == 0 || (parts && inv && weights)) && (!mat || self_rows)),
                "dyt_seam_f32 failed: the expert rows need their index and weights");
    if (rows <= 0) return 0;
    SeamArgs a{mode, y, y2, weight_a, weight_b, mult, eps,
               CombineArgs{parts, inv, mat, weights, top, self_rows, shared_rows, gate_rows, ldg, gate_off, nullptr, width},
               alpha1, w1, b1, x, alpha2, w2, b2, h, width};
    const int by = rows <= 32 ? (width + 511) / 512 < 8 ? (width + 511) / 512 : 8 : 1;
    PGK_CUDA(launch(dyt_seam_kernel, dim3(rows, by), dim3(256), 0, (cudaStream_t)stream, a));
    return 0;
}

int pgk_seq_gated_prep(float* proj, int ld, int tokens, int heads, int dim, int q_off, int f_off, const float* f_bias,
                       const float* lower, void* stream) {
    PGK_REQUIRE(heads > 0 && dim > 0, "seq_gated_prep failed: invalid head layout");
    if (tokens <= 0) return 0;
    PGK_CUDA(launch(gated_prep_kernel, dim3(tokens, (2 * heads + 3) / 4), dim3(128), 0, (cudaStream_t)stream, proj, ld, heads, dim,
                    q_off, f_off, f_bias, lower));
    return 0;
}

int pgk_seq_delta_prep(float* qk_rows, int ldqk, int q_off, int k_off, float* proj, int ld, int beta_off, int a_off,
                       const float* A_log, const float* dt_bias, int tokens, int heads, int qk_heads, int dim, float q_mult,
                       void* stream) {
    PGK_REQUIRE(heads > 0 && qk_heads > 0 && heads % qk_heads == 0 && dim > 0 && A_log && dt_bias, "seq_delta_prep failed: invalid head layout");
    if (tokens <= 0) return 0;
    DeltaPrepArgs a{qk_rows, ldqk, q_off, k_off, proj, ld, beta_off, a_off, A_log, dt_bias, heads, qk_heads, dim, q_mult};
    PGK_CUDA(launch(delta_prep_kernel, dim3(tokens, (2 * qk_heads + 1 + 3) / 4), dim3(128), 0, (cudaStream_t)stream, a));
    return 0;
}

int pgk_seq_gated_recurrence(int delta, const float* q, int ldq, int q_off, const float* k, int ldk, int k_off, const float* a,
                             int lda, int a_off, const float* beta, int ldb, int b_off, const float* v, int ldv, int v_off,
                             float* out, int ldo, float* state, const int32_t* seqs, int n_seqs, int heads, int qk_heads, int dim,
                             int vdim, void* stream) {
    PGK_REQUIRE(heads > 0 && qk_heads > 0 && heads % qk_heads == 0 && dim > 0 && dim <= 256 && vdim > 0,
                "seq_gated_recurrence failed: %d heads over %d query/key heads of %d (at most 256) x %d", heads, qk_heads, dim, vdim);
    PGK_REQUIRE(q && a && v && out && state && (!delta || (k && beta)), "seq_gated_recurrence failed: a missing operand");
    if (n_seqs <= 0) return 0;
    GatedArgs g{q, ldq, q_off, k, ldk, k_off, a, lda, a_off, beta, ldb, b_off, v, ldv, v_off, out, ldo, state, (const int4*)seqs,
                heads, qk_heads, dim, vdim};
    return delta ? run_gated<true>(g, n_seqs, (cudaStream_t)stream) : run_gated<false>(g, n_seqs, (cudaStream_t)stream);
}

}  // extern "C"
