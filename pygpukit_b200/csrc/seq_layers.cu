// seq_layers.cu -- the row-wise pieces of the token-major models, all in float32: embedding rows, the fused
// "sum the sublayer's parts -> LayerNorm -> add to the residual" step, row gather + LayerNorm (final norm of the wanted
// rows), and the mixture-of-experts router (softmax over all experts, group-limited top-k, renormalised weights) with the
// per-expert row lists the grouped GEMM consumes; and the RMS norm of rows (weight with an offset, optional second summand
// that is written back, optional accumulation into the output) that the pre-norm blocks are built from.
#include "common.cuh"
#include "../../include/pgk_b200.h"

using namespace pgk;

namespace {

template <typename TW> __device__ __forceinline__ float wload(const TW* p);
template <> __device__ __forceinline__ float wload<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float wload<uint16_t>(const uint16_t* p) { return bf16_bits_to_f32(*p); }

template <typename TW>
__global__ void __launch_bounds__(256) embed_rows_kernel(const TW* table, const int* tok, float* x, int W, int vocab) {
    const int t = blockIdx.x;
    int id = tok[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const TW* src = table + (size_t)id * W;
    const int i0 = (blockIdx.y * 256 + threadIdx.x) * 4;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = i0 + j < W ? wload<TW>(src + i0 + j) : 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (i0 + j < W) x[(size_t)t * W + i0 + j] = v[j];
}

__device__ __forceinline__ float block_sum256(float v, float* red) {
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

// y = base[src] + sum_k w[t, k] * parts[inv[t, k]];  LayerNorm(y) * gamma + beta;  ADD: x[t] += that, else out[t] = that
struct NormArgs {
    const float* base; const int* src_rows;          // base may be NULL; src_rows gathers base rows (NULL: t)
    const float* parts; const int* inv; const float* w; int top;
    const float* gamma; const float* beta; float eps;
    float* out; int W; int add;
};

constexpr int TOPMAX = 64;          // (token, slot) rows staged in shared memory; beyond that they are re-read

__global__ void __launch_bounds__(256) combine_norm_kernel(NormArgs a) {
    extern __shared__ float y[];
    __shared__ float red[8];
    __shared__ float wk[TOPMAX];
    __shared__ long long pk[TOPMAX];
    const int t = blockIdx.x;
    const size_t srow = a.src_rows ? (size_t)a.src_rows[t] : (size_t)t;
    const int top = a.top;
    if (threadIdx.x < top && threadIdx.x < TOPMAX) {
        wk[threadIdx.x] = a.w[(size_t)t * top + threadIdx.x];
        pk[threadIdx.x] = (long long)a.inv[(size_t)t * top + threadIdx.x] * a.W;
    }
    if (top > 0) __syncthreads();
    float s = 0.f;
    for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
        float v = 0.f;
        const int ks = top < TOPMAX ? top : TOPMAX;
#pragma unroll 8
        for (int k = 0; k < ks; ++k) v = fmaf(wk[k], a.parts[pk[k] + i], v);
        for (int k = TOPMAX; k < top; ++k)
            v = fmaf(a.w[(size_t)t * top + k], a.parts[(size_t)a.inv[(size_t)t * top + k] * a.W + i], v);
        if (a.base) v += a.base[srow * a.W + i];
        y[i] = v;
        s += v;
    }
    const float mean = block_sum256(s, red) / (float)a.W;
    float q = 0.f;
    for (int i = threadIdx.x; i < a.W; i += blockDim.x) { const float d = y[i] - mean; q = fmaf(d, d, q); }
    const float var = block_sum256(q, red) / (float)a.W;
    const float inv = 1.f / sqrtf(var + a.eps);
    for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
        const float v = (y[i] - mean) * inv * a.gamma[i] + (a.beta ? a.beta[i] : 0.f);
        float* o = a.out + (size_t)t * a.W + i;
        *o = a.add ? *o + v : v;
    }
}

// ---------------------------------------------------------------- RMS norm of rows
// v = x[src] (+ add[t]);  sum_out[t] = v (when given);  r = v / sqrt(mean(v^2) + eps) * (w_off + w);
// accumulate: out[t] += r, else out[t] = r.  `out` may be `x` (the row is staged in shared memory first).
struct RmsArgs {
    const float* x; const int* src_rows; const float* add; float* sum_out;
    const float* w; float w_off, eps;
    float* out; int W; int accumulate;
};

__global__ void __launch_bounds__(256) rms_norm_rows_kernel(RmsArgs a) {
    extern __shared__ float y[];
    __shared__ float red[8];
    const int t = blockIdx.x;
    const size_t srow = a.src_rows ? (size_t)a.src_rows[t] : (size_t)t;
    float q = 0.f;
    for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
        float v = a.x[srow * a.W + i];
        if (a.add) v += a.add[(size_t)t * a.W + i];
        y[i] = v;
        q = fmaf(v, v, q);
    }
    const float inv = 1.f / sqrtf(block_sum256(q, red) / (float)a.W + a.eps);
    for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
        const float v = y[i];
        if (a.sum_out) a.sum_out[(size_t)t * a.W + i] = v;
        const float r = v * inv * (a.w_off + a.w[i]);
        float* o = a.out + (size_t)t * a.W + i;
        *o = a.accumulate ? *o + r : r;
    }
}

// Two norms in one pass over the row, for the seam between two pre-norm blocks: x[t] += rms(y[t]) * (off1 + w1) (a
// normalised branch joins the residual stream), then (+ add[t], written back into x as well) h[t] = rms(x[t]) * (off2 + w2)
// is the next block's input.
struct RmsSeamArgs {
    const float* y; const float* w1; float off1;
    float* x; const float* add;
    const float* w2; float off2, eps;
    float* h; int W;
};

__global__ void __launch_bounds__(256) rms_seam_kernel(RmsSeamArgs a) {
    extern __shared__ float row[];
    __shared__ float red[8];
    const int t = blockIdx.x;
    const size_t o = (size_t)t * a.W;
    float q = 0.f;
    for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
        const float v = a.y[o + i];
        row[i] = v;
        q = fmaf(v, v, q);
    }
    const float inv1 = 1.f / sqrtf(block_sum256(q, red) / (float)a.W + a.eps);
    q = 0.f;
    for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
        float v = a.x[o + i] + row[i] * inv1 * (a.off1 + a.w1[i]);
        if (a.add) v += a.add[o + i];
        a.x[o + i] = v;
        row[i] = v;
        q = fmaf(v, v, q);
    }
    const float inv2 = 1.f / sqrtf(block_sum256(q, red) / (float)a.W + a.eps);
    for (int i = threadIdx.x; i < a.W; i += blockDim.x) a.h[o + i] = row[i] * inv2 * (a.off2 + a.w2[i]);
}

// x[t] = rms(table[tokens[t]]) * (off + w), copied to keep[t] as well when given: embedding, its norm and the kept copy
template <typename TW>
__global__ void __launch_bounds__(256) embed_norm_rows_kernel(const TW* table, const int* tok, const float* w, float off, float eps,
                                                              float* x, float* keep, int W, int vocab) {
    extern __shared__ float row[];
    __shared__ float red[8];
    const int t = blockIdx.x;
    int id = tok[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const TW* src = table + (size_t)id * W;
    float q = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float v = wload<TW>(src + i);
        row[i] = v;
        q = fmaf(v, v, q);
    }
    const float inv = 1.f / sqrtf(block_sum256(q, red) / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float v = row[i] * inv * (off + w[i]);
        x[(size_t)t * W + i] = v;
        if (keep) keep[(size_t)t * W + i] = v;
    }
}

// ---------------------------------------------------------------- router
struct RouteArgs {
    const float* z; int ldz; int T, E, top, gcount, gkeep;
    int* idx; float* wt; int* rank; int* counts;
};

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

constexpr int ROUTE_WARPS = 4;       // tokens per block, one warp each

__global__ void __launch_bounds__(ROUTE_WARPS * 32) moe_route_kernel(RouteArgs a) {
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= a.T) return;
    float* s = sm + (size_t)warp * (2 * a.E + a.gcount);     // [E] scores
    float* gs = s + a.E;                                      // [gcount]
    int* open = (int*)(gs + a.gcount);                        // [E] 1 = may still be chosen
    const float* z = a.z + (size_t)t * a.ldz;
    float mx = -INFINITY;
    for (int e = lane; e < a.E; e += 32) { const float v = z[e]; s[e] = v; mx = fmaxf(mx, v); }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < a.E; e += 32) { const float p = expf(s[e] - mx); s[e] = p; sum += p; }
    sum = warp_sum(sum);
    for (int e = lane; e < a.E; e += 32) { s[e] = s[e] / sum; open[e] = 1; }
    __syncwarp();
    if (a.gcount > 1 && a.gkeep < a.gcount) {
        const int per = a.E / a.gcount;
        for (int g = lane; g < a.gcount; g += 32) {
            float b = -1.f;
            for (int j = 0; j < per; ++j) b = fmaxf(b, s[g * per + j]);
            gs[g] = b;
        }
        for (int e = lane; e < a.E; e += 32) open[e] = 0;
        __syncwarp();
        for (int it = 0; it < a.gkeep; ++it) {
            float bv = -2.f; int bi = 0x7fffffff;
            for (int g = lane; g < a.gcount; g += 32)
                if (gs[g] > bv) { bv = gs[g]; bi = g; }
            warp_argmax(bv, bi);
            if (lane == 0) gs[bi] = -3.f;
            for (int j = lane; j < per; j += 32) open[bi * per + j] = 1;
            __syncwarp();
        }
    }
    float wsum = 0.f, mine = 0.f; int mine_i = 0;
    for (int k = 0; k < a.top; ++k) {
        float bv = -1.f; int bi = 0x7fffffff;
        for (int e = lane; e < a.E; e += 32)
            if (open[e] && s[e] > bv) { bv = s[e]; bi = e; }
        warp_argmax(bv, bi);
        if (lane == 0) open[bi] = 0;
        __syncwarp();
        wsum += bv;
        if (lane == k % 32 && k < 32) { mine = bv; mine_i = bi; }
        if (k >= 32 && lane == 0) {        // more than 32 slots: lane 0 writes unnormalised, fixed below
            a.idx[(size_t)t * a.top + k] = bi; a.wt[(size_t)t * a.top + k] = bv;
        }
    }
    const float norm = wsum + 1e-20f;
    if (lane < a.top && lane < 32) {
        const size_t o = (size_t)t * a.top + lane;
        a.idx[o] = mine_i;
        a.wt[o] = mine / norm;
        if (a.counts) a.rank[o] = atomicAdd(&a.counts[mine_i], 1);
    }
    if (a.top > 32 && lane == 0)
        for (int k = 32; k < a.top; ++k) {
            const size_t o = (size_t)t * a.top + k;
            a.wt[o] = a.wt[o] / norm;
            if (a.counts) a.rank[o] = atomicAdd(&a.counts[a.idx[o]], 1);
        }
}

// offsets = exclusive scan of counts (which are cleared for the next use); rows of expert e = offsets[e] .. offsets[e+1];
// perm[row] = token, inv[t * top + k] = row
__global__ void __launch_bounds__(1024) moe_lists_kernel(int* counts, int* offsets, const int* idx, const int* rank, int* perm,
                                                        int* inv, int E, int n, int top) {
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < E; ++e) { offsets[e] = acc; acc += counts[e]; counts[e] = 0; }
        offsets[E] = acc;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int r = offsets[idx[i]] + rank[i];
        perm[r] = i / top;
        inv[i] = r;
    }
}

}  // namespace

extern "C" {

int pgk_embed_rows_f32(const void* table, int wdt, const int32_t* tokens, float* x, int n, int width, int vocab, void* stream) {
    PGK_REQUIRE(wdt == 0 || wdt == 2, "embed_rows_f32 failed: table must be float32 (0) or bfloat16 (2), got %d", wdt);
    if (n <= 0) return 0;
    if (wdt == 2) PGK_CUDA(launch(embed_rows_kernel<uint16_t>, dim3(n, (width + 1023) / 1024), dim3(256), 0, (cudaStream_t)stream, (const uint16_t*)table, tokens, x, width, vocab));
    else PGK_CUDA(launch(embed_rows_kernel<float>, dim3(n, (width + 1023) / 1024), dim3(256), 0, (cudaStream_t)stream, (const float*)table, tokens, x, width, vocab));
    return 0;
}

int pgk_combine_layernorm_f32(const float* base, const int32_t* src_rows, const float* parts, const int32_t* inv,
                              const float* weights, int top, const float* gamma, const float* beta, float eps, float* out,
                              int rows, int width, int add, void* stream) {
    PGK_REQUIRE(width > 0 && width * 4 <= 160 * 1024, "combine_layernorm_f32 failed: width %d out of range", width);
    PGK_REQUIRE(top == 0 || (parts && inv && weights), "combine_layernorm_f32 failed: parts need their index and weights");
    if (rows <= 0) return 0;
    NormArgs a{base, src_rows, parts, inv, weights, top, gamma, beta, eps, out, width, add};
    const size_t smem = (size_t)width * 4;
    static bool configured = false;
    if (smem > 40 * 1024 && !configured) {          // dynamic + static shared memory pass 48 KB a little earlier
        PGK_CUDA(cudaFuncSetAttribute(combine_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        configured = true;
    }
    PGK_CUDA(launch(combine_norm_kernel, dim3(rows), dim3(256), smem, (cudaStream_t)stream, a));
    return 0;
}

int pgk_rms_norm_rows_f32(const float* x, const int32_t* src_rows, const float* add, float* sum_out, const float* weight,
                          float weight_offset, float eps, float* out, int rows, int width, int accumulate, void* stream) {
    PGK_REQUIRE(width > 0 && width * 4 <= 160 * 1024, "rms_norm_rows_f32 failed: width %d out of range", width);
    PGK_REQUIRE(!(sum_out && src_rows), "rms_norm_rows_f32 failed: the sum is written back only without a row gather");
    if (rows <= 0) return 0;
    RmsArgs a{x, src_rows, add, sum_out, weight, weight_offset, eps, out, width, accumulate};
    const size_t smem = (size_t)width * 4;
    static bool configured = false;
    if (smem > 40 * 1024 && !configured) {          // dynamic + static shared memory pass 48 KB a little earlier
        PGK_CUDA(cudaFuncSetAttribute(rms_norm_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        configured = true;
    }
    PGK_CUDA(launch(rms_norm_rows_kernel, dim3(rows), dim3(256), smem, (cudaStream_t)stream, a));
    return 0;
}

int pgk_rms_norm_seam_f32(const float* y, const float* weight1, float offset1, float* x, const float* add, const float* weight2,
                          float offset2, float eps, float* h, int rows, int width, void* stream) {
    PGK_REQUIRE(width > 0 && width * 4 <= 160 * 1024, "rms_norm_seam_f32 failed: width %d out of range", width);
    if (rows <= 0) return 0;
    RmsSeamArgs a{y, weight1, offset1, x, add, weight2, offset2, eps, h, width};
    const size_t smem = (size_t)width * 4;
    static bool configured = false;
    if (smem > 40 * 1024 && !configured) {
        PGK_CUDA(cudaFuncSetAttribute(rms_seam_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        configured = true;
    }
    PGK_CUDA(launch(rms_seam_kernel, dim3(rows), dim3(256), smem, (cudaStream_t)stream, a));
    return 0;
}

int pgk_embed_norm_rows_f32(const void* table, int wdt, const int32_t* tokens, const float* weight, float weight_offset, float eps,
                            float* x, float* keep, int n, int width, int vocab, void* stream) {
    PGK_REQUIRE(wdt == 0 || wdt == 2, "embed_norm_rows_f32 failed: table must be float32 (0) or bfloat16 (2), got %d", wdt);
    PGK_REQUIRE(width > 0 && width * 4 <= 160 * 1024, "embed_norm_rows_f32 failed: width %d out of range", width);
    if (n <= 0) return 0;
    const size_t smem = (size_t)width * 4;
    static bool configured = false;
    if (smem > 40 * 1024 && !configured) {
        PGK_CUDA(cudaFuncSetAttribute(embed_norm_rows_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        PGK_CUDA(cudaFuncSetAttribute(embed_norm_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        configured = true;
    }
    if (wdt == 2) PGK_CUDA(launch(embed_norm_rows_kernel<uint16_t>, dim3(n), dim3(256), smem, (cudaStream_t)stream, (const uint16_t*)table, tokens, weight, weight_offset, eps, x, keep, width, vocab));
    else PGK_CUDA(launch(embed_norm_rows_kernel<float>, dim3(n), dim3(256), smem, (cudaStream_t)stream, (const float*)table, tokens, weight, weight_offset, eps, x, keep, width, vocab));
    return 0;
}

int pgk_moe_route_grouped(const float* logits, int ld, int tokens, int experts, int top, int group_count, int group_keep,
                          int32_t* idx, float* weights, int32_t* rank, int32_t* counts, void* stream) {
    PGK_REQUIRE(experts > 0 && top > 0 && top <= experts, "moe_route_grouped failed: top %d of %d experts", top, experts);
    if (group_count < 1) group_count = 1;
    PGK_REQUIRE(experts % group_count == 0 && group_keep >= 1, "moe_route_grouped failed: %d experts in %d groups (keep %d)", experts, group_count, group_keep);
    PGK_REQUIRE(group_count == 1 || group_keep >= group_count || (experts / group_count) * group_keep >= top,
                "moe_route_grouped failed: %d kept groups hold fewer than top = %d experts", group_keep, top);
    if (tokens <= 0) return 0;
    RouteArgs a{logits, ld, tokens, experts, top, group_count, group_keep, idx, weights, rank, counts};
    const size_t smem = (size_t)ROUTE_WARPS * (2 * experts + group_count) * 4;
    PGK_REQUIRE(smem <= 48 * 1024, "moe_route_grouped failed: too many experts (%d)", experts);
    PGK_CUDA(launch(moe_route_kernel, dim3((tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem,
                    (cudaStream_t)stream, a));
    return 0;
}

int pgk_moe_row_lists(int32_t* counts, int32_t* offsets, const int32_t* idx, const int32_t* rank, int32_t* perm, int32_t* inv,
                      int experts, int tokens, int top, void* stream) {
    if (tokens <= 0) return 0;
    PGK_CUDA(launch(moe_lists_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, counts, offsets, idx, rank, perm, inv, experts,
                    tokens * top, top));
    return 0;
}

}  // extern "C"
