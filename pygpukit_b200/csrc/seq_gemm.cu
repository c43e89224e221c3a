// seq_gemm.cu -- C[m, n] = sum_k A[row(m), k] * W[g][n, k] for the token-major ("ragged batch") models: float32
// activations, weights [N, K] K-contiguous in bfloat16 or float32, float32 accumulation and output.
//
//   * many rows (prompts): 64 x 64 x 32 tiles, four warps; bfloat16 weights run on the tensor cores (mma.sync m16n8k16,
//     the activation tile is rounded to bfloat16 while it is staged), float32 weights on FMAs with no reduced-precision
//     mode anywhere;
//   * few rows (decoding): a warp per output column streams its weight row once with 128-bit loads and serves up to
//     eight rows of A held in shared memory;
//   * groups: `group_off` [E + 1] cuts the rows into E consecutive runs, run e uses weight matrix e (mixture of experts:
//     the rows are (token, slot) pairs sorted by expert); `a_rows` gathers the rows of A, so the tokens are never copied;
//   * epilogues: plain; gate/up pairs (W holds gate_j in row 2j and up_j in row 2j + 1, the output is silu(gate) * up,
//     [M, N / 2]); scale then tanh cap (the logit head); clamped gate/up pairs g = min(gate, limit), u = clamp(up, +-limit),
//     output g sigmoid(alpha g) (u + 1); C += column vector * product (layer scale and residual add in one pass);
//     gelu_tanh(product) * gathered table entry (per-layer token inputs);
//   * batches: grid.z can also walk `batch` independent products whose A columns, matrices and C columns are a fixed number
//     of elements apart (one product per attention head on slices of the same rows).
#include "common.cuh"
#include "../../include/pgk_b200.h"

using namespace pgk;

namespace {

struct GemmArgs {
    const float* A;
    const int* a_rows;
    const void* W;
    float* C;
    const int* group_off;
    const int* row_group;     // few-row form: weight matrix of every row (NULL: matrix 0)
    long long w_stride;       // elements between the weight matrices of consecutive groups
    int lda, ldc, M, N, K;
    float scale, cap;
    const float* colv;        // epilogue 4: [N] factors of the accumulated product
    const void* aux;          // epilogue 5: table [*, aux_ld] (float32 or bfloat16), entry (aux_rows[m], aux_off + n)
    const int* aux_rows;
    int aux_ld, aux_off, aux_dt;
    long long a_z, c_z;       // batches: elements between the A columns / C columns of consecutive products
};

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float aux_at(const GemmArgs& a, int row, int col) {
    const size_t i = (size_t)a.aux_rows[row] * a.aux_ld + a.aux_off + col;
    return a.aux_dt == 2 ? bf16_bits_to_f32(((const uint16_t*)a.aux)[i]) : ((const float*)a.aux)[i];
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

template <int EPI>
__device__ __forceinline__ void store_pair(const GemmArgs& a, int row, int col, float c0, float c1) {
    // (row, col) and (row, col + 1), col even
    if (EPI == 1) {
        if (col + 1 < a.N) a.C[(size_t)row * a.ldc + (col >> 1)] = silu_f(c0) * c1;
        return;
    }
    if (EPI == 3) {          // scale = alpha, cap = limit
        if (col + 1 < a.N) {
            const float g = fminf(c0, a.cap), u = fminf(fmaxf(c1, -a.cap), a.cap);
            a.C[(size_t)row * a.ldc + (col >> 1)] = g / (1.f + expf(-a.scale * g)) * (u + 1.f);
        }
        return;
    }
    if (EPI == 2) {
        c0 *= a.scale; c1 *= a.scale;
        if (a.cap > 0.f) { c0 = a.cap * tanhf(c0 / a.cap); c1 = a.cap * tanhf(c1 / a.cap); }
    }
    if (EPI == 6) {          // squared ReLU
        c0 = fmaxf(c0, 0.f); c1 = fmaxf(c1, 0.f);
        c0 *= c0; c1 *= c1;
    }
    float* p = a.C + (size_t)row * a.ldc + col;
    if (EPI == 4) {
        if (col < a.N) p[0] = fmaf(a.colv[col], c0, p[0]);
        if (col + 1 < a.N) p[1] = fmaf(a.colv[col + 1], c1, p[1]);
        return;
    }
    if (EPI == 5) {
        if (col < a.N) p[0] = gelu_tanh_f(c0) * aux_at(a, row, col);
        if (col + 1 < a.N) p[1] = gelu_tanh_f(c1) * aux_at(a, row, col + 1);
        return;
    }
    if (col < a.N) p[0] = c0;
    if (col + 1 < a.N) p[1] = c1;
}

constexpr int BM = 64, BN = 64, BK = 32;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem_row)));
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// ---------------------------------------------------------------- many rows, bfloat16 weights: tensor cores
template <int EPI>
__global__ void __launch_bounds__(128) gemm_rows_bf16_kernel(GemmArgs a) {
    const int e = blockIdx.z;
    a.A += (size_t)e * a.a_z;
    a.C += (size_t)e * a.c_z;
    const int m_begin = a.group_off ? a.group_off[e] : 0;
    const int m_end = a.group_off ? a.group_off[e + 1] : a.M;
    const int m0 = m_begin + blockIdx.y * BM;
    if (m0 >= m_end) return;
    const int n0 = blockIdx.x * BN;
    const uint16_t* W = (const uint16_t*)a.W + (size_t)e * a.w_stride;

    __shared__ __align__(16) uint16_t As[2][BM][BK + 8];
    __shared__ __align__(16) uint16_t Ws[2][BN][BK + 8];
    __shared__ int rows[BM];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < BM) {
        const int r = m0 + tid;
        rows[tid] = r < m_end ? (a.a_rows ? a.a_rows[r] : r) : -1;
    }
    __syncthreads();
    const bool avec = (a.K % 4 == 0) && (a.lda % 4 == 0) && (((uintptr_t)a.A & 15) == 0);
    const bool wvec = (a.K % 8 == 0) && (((uintptr_t)W & 15) == 0);

    float4 ra[4];
    uint4 rw[2];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 128, r = idx >> 3, c = (idx & 7) * 4, gr = rows[r], k = k0 + c;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gr >= 0) {
                const float* p = a.A + (size_t)gr * a.lda + k;
                if (avec && k + 3 < a.K) v = *(const float4*)p;
                else {
                    if (k < a.K) v.x = p[0];
                    if (k + 1 < a.K) v.y = p[1];
                    if (k + 2 < a.K) v.z = p[2];
                    if (k + 3 < a.K) v.w = p[3];
                }
            }
            ra[i] = v;
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + i * 128, r = idx >> 2, c = (idx & 3) * 8, n = n0 + r, k = k0 + c;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (n < a.N) {
                const uint16_t* p = W + (size_t)n * a.K + k;
                if (wvec && k + 7 < a.K) v = *(const uint4*)p;
                else {
                    uint16_t t[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) t[j] = (k + j < a.K) ? p[j] : (uint16_t)0;
                    v.x = t[0] | ((uint32_t)t[1] << 16); v.y = t[2] | ((uint32_t)t[3] << 16);
                    v.z = t[4] | ((uint32_t)t[5] << 16); v.w = t[6] | ((uint32_t)t[7] << 16);
                }
            }
            rw[i] = v;
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 128, r = idx >> 3, c = (idx & 7) * 4;
            uint2 v = make_uint2(pack_bf16x2(ra[i].x, ra[i].y), pack_bf16x2(ra[i].z, ra[i].w));
            *(uint2*)&As[buf][r][c] = v;
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + i * 128, r = idx >> 2, c = (idx & 3) * 8;
            *(uint4*)&Ws[buf][r][c] = rw[i];
        }
    };

    float acc[2][4][4] = {};
    const int wm = warp >> 1, wn = warp & 1, g = lane >> 2, tg = lane & 3;
    const int nk = (a.K + BK - 1) / BK;
    fetch(0);
    stash(0);
    __syncthreads();
    for (int kt = 0; kt < nk; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < nk) fetch((kt + 1) * BK);
#pragma unroll
        for (int kk = 0; kk < BK; kk += 16) {
            // fragments by ldmatrix (rows are 80 bytes apart: 16-byte aligned and conflict-free)
            uint32_t af[2][4], bf[4][2];
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)      // 16 x 16 of A: lanes 0-15 name rows 0-15 at k, lanes 16-31 the same rows at k + 8
                ldmatrix_x4(af[mi], &As[buf][wm * 32 + mi * 16 + (lane & 15)][kk + ((lane >> 4) << 3)]);
#pragma unroll
            for (int nj = 0; nj < 2; ++nj) {    // 16 columns x 16 k of W: (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
                uint32_t r[4];
                ldmatrix_x4(r, &Ws[buf][wn * 32 + nj * 16 + (lane & 7) + ((lane >> 4) << 3)][kk + (((lane >> 3) & 1) << 3)]);
                bf[2 * nj][0] = r[0]; bf[2 * nj][1] = r[1]; bf[2 * nj + 1][0] = r[2]; bf[2 * nj + 1][1] = r[3];
            }
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int ni = 0; ni < 4; ++ni) mma_bf16(acc[mi][ni], af[mi], bf[ni]);
        }
        if (kt + 1 < nk) stash(buf ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) {
            const int r = m0 + wm * 32 + mi * 16 + g, c = n0 + wn * 32 + ni * 8 + 2 * tg;
            if (r < m_end) store_pair<EPI>(a, r, c, acc[mi][ni][0], acc[mi][ni][1]);
            if (r + 8 < m_end) store_pair<EPI>(a, r + 8, c, acc[mi][ni][2], acc[mi][ni][3]);
        }
}

// ---------------------------------------------------------------- many rows, float32 weights: FMAs, summed in k order
template <int EPI>
__global__ void __launch_bounds__(128) gemm_rows_f32_kernel(GemmArgs a) {
    const int e = blockIdx.z;
    a.A += (size_t)e * a.a_z;
    a.C += (size_t)e * a.c_z;
    const int m_begin = a.group_off ? a.group_off[e] : 0;
    const int m_end = a.group_off ? a.group_off[e + 1] : a.M;
    const int m0 = m_begin + blockIdx.y * BM;
    if (m0 >= m_end) return;
    const int n0 = blockIdx.x * BN;
    const float* W = (const float*)a.W + (size_t)e * a.w_stride;
    constexpr int FK = 16;
    __shared__ float As[FK][BM + 4];
    __shared__ float Ws[FK][BN + 4];
    __shared__ int rows[BM];
    const int tid = threadIdx.x;
    if (tid < BM) {
        const int r = m0 + tid;
        rows[tid] = r < m_end ? (a.a_rows ? a.a_rows[r] : r) : -1;
    }
    __syncthreads();
    const int ty = tid >> 4, tx = tid & 15;          // 8 rows x 4 columns per thread
    float acc[8][4] = {};
    for (int k0 = 0; k0 < a.K; k0 += FK) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int idx = tid + i * 128, r = idx >> 4, c = idx & 15, k = k0 + c;
            const int gr = rows[r];
            As[c][r] = (gr >= 0 && k < a.K) ? a.A[(size_t)gr * a.lda + k] : 0.f;
            const int n = n0 + r;
            Ws[c][r] = (n < a.N && k < a.K) ? W[(size_t)n * a.K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < FK; ++k) {
            float av[8], wv[4];
#pragma unroll
            for (int i = 0; i < 8; ++i) av[i] = As[k][ty * 8 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = m0 + ty * 8 + i;
        if (r >= m_end) continue;
        store_pair<EPI>(a, r, n0 + tx * 4, acc[i][0], acc[i][1]);
        store_pair<EPI>(a, r, n0 + tx * 4 + 2, acc[i][2], acc[i][3]);
    }
}

// ---------------------------------------------------------------- few rows: one warp per output column (pair)
// Block = 4 .. 16 warps; the block's rows of A (<= RMAX, all using the same weight matrix) sit in shared memory as float32;
// a warp owns two consecutive output columns (a gate/up pair under EPI 1), reads their weight rows once with 128-bit
// loads and forms the dot products of every row.  grid = (column pairs / 8, row blocks).
constexpr int RMAX = 8;

template <typename TW> struct WLoad;
template <> struct WLoad<uint16_t> {
    static constexpr int VEC = 8;
    static __device__ __forceinline__ void unpack(const uint4& v, float (&w)[8]) {
        w[0] = bf16lo(v.x); w[1] = bf16hi(v.x); w[2] = bf16lo(v.y); w[3] = bf16hi(v.y);
        w[4] = bf16lo(v.z); w[5] = bf16hi(v.z); w[6] = bf16lo(v.w); w[7] = bf16hi(v.w);
    }
    static __device__ __forceinline__ float one(const uint16_t* p) { return bf16_bits_to_f32(*p); }
};
template <> struct WLoad<float> {
    static constexpr int VEC = 4;
    static __device__ __forceinline__ void unpack(const uint4& v, float (&w)[8]) {
        w[0] = __uint_as_float(v.x); w[1] = __uint_as_float(v.y); w[2] = __uint_as_float(v.z); w[3] = __uint_as_float(v.w);
        w[4] = w[5] = w[6] = w[7] = 0.f;
    }
    static __device__ __forceinline__ float one(const float* p) { return *p; }
};

constexpr int FEW_MAX_WARPS = 16;  // warps (= column pairs) per block: 4 .. 16, more when the staged rows take much shared memory
constexpr int FEW_UN = 4;         // 128-bit loads per weight row in flight per lane

template <typename TW, int EPI, bool ROUND>
__global__ void __launch_bounds__(FEW_MAX_WARPS * 32) gemm_few_rows_kernel(GemmArgs a, int rows_per_block) {
    extern __shared__ __align__(16) float xs[];                 // [rows][K]
    const int r0 = blockIdx.y * rows_per_block;
    const int nr = min(rows_per_block, a.M - r0);
    const int grp = a.row_group ? a.row_group[r0] : (int)blockIdx.z;
    if (grp < 0) return;                                        // a row without a matrix (its output is formed elsewhere)
    a.A += (size_t)blockIdx.z * a.a_z;
    a.C += (size_t)blockIdx.z * a.c_z;
    const TW* W = (const TW*)a.W + (size_t)grp * a.w_stride;
    constexpr int VEC = WLoad<TW>::VEC;
    const bool vec = (a.K % VEC == 0) && (((uintptr_t)W & 15) == 0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c0 = (blockIdx.x * (blockDim.x >> 5) + warp) * 2;
    const bool live = c0 < a.N;
    const bool two = c0 + 1 < a.N;
    const TW* w0 = W + (size_t)(live ? c0 : 0) * a.K;
    const TW* w1 = W + (size_t)(two ? c0 + 1 : (live ? c0 : 0)) * a.K;
    // the first weight loads do not depend on the activations: issue them before staging x
    uint4 ru[FEW_UN], rv[FEW_UN];
    const int kstep = 32 * VEC;
    if (vec) {
#pragma unroll
        for (int j = 0; j < FEW_UN; ++j) {
            const int k = lane * VEC + j * kstep;
            ru[j] = rv[j] = make_uint4(0u, 0u, 0u, 0u);
            if (live && k < a.K) { ru[j] = ldg_stream(w0 + k); rv[j] = ldg_stream(w1 + k); }
        }
    }
    const bool xvec = (a.K % 4 == 0) && (a.lda % 4 == 0) && (((uintptr_t)a.A & 15) == 0);
    if (xvec) {
        const int k4 = a.K >> 2;
        for (int i = threadIdx.x; i < nr * k4; i += blockDim.x) {
            const int r = i / k4, k = (i - r * k4) * 4;
            const int gr = a.a_rows ? a.a_rows[r0 + r] : r0 + r;
            float4 v = *(const float4*)(a.A + (size_t)gr * a.lda + k);
            if (ROUND) { v.x = round_bf16(v.x); v.y = round_bf16(v.y); v.z = round_bf16(v.z); v.w = round_bf16(v.w); }
            *(float4*)(xs + r * a.K + k) = v;
        }
    } else {
        for (int i = threadIdx.x; i < nr * a.K; i += blockDim.x) {
            const int r = i / a.K, k = i - r * a.K;
            const int gr = a.a_rows ? a.a_rows[r0 + r] : r0 + r;
            const float v = a.A[(size_t)gr * a.lda + k];
            xs[i] = ROUND ? round_bf16(v) : v;
        }
    }
    __syncthreads();
    if (!live) return;
    float acc0[RMAX] = {}, acc1[RMAX] = {};
    if (vec) {
        for (int kb = 0; kb < a.K; kb += FEW_UN * kstep) {
            uint4 cu[FEW_UN], cv[FEW_UN];
#pragma unroll
            for (int j = 0; j < FEW_UN; ++j) { cu[j] = ru[j]; cv[j] = rv[j]; }
            const int kn = kb + FEW_UN * kstep;
            if (kn < a.K) {
#pragma unroll
                for (int j = 0; j < FEW_UN; ++j) {
                    const int k = kn + lane * VEC + j * kstep;
                    if (k < a.K) { ru[j] = ldg_stream(w0 + k); rv[j] = ldg_stream(w1 + k); }
                }
            }
#pragma unroll
            for (int j = 0; j < FEW_UN; ++j) {
                const int k = kb + lane * VEC + j * kstep;
                if (k >= a.K) continue;
                float u[8], v[8];
                WLoad<TW>::unpack(cu[j], u);
                WLoad<TW>::unpack(cv[j], v);
#pragma unroll
                for (int r = 0; r < RMAX; ++r) {
                    if (r < nr) {
                        float x[8];
                        *(float4*)&x[0] = *(const float4*)(xs + r * a.K + k);
                        if (VEC == 8) *(float4*)&x[4] = *(const float4*)(xs + r * a.K + k + 4);
#pragma unroll
                        for (int q = 0; q < VEC; ++q) {
                            acc0[r] = fmaf(x[q], u[q], acc0[r]);
                            acc1[r] = fmaf(x[q], v[q], acc1[r]);
                        }
                    }
                }
            }
        }
    } else {
        for (int k = lane; k < a.K; k += 32) {
            const float u = WLoad<TW>::one(w0 + k), v = WLoad<TW>::one(w1 + k);
#pragma unroll
            for (int r = 0; r < RMAX; ++r)
                if (r < nr) {
                    acc0[r] = fmaf(xs[r * a.K + k], u, acc0[r]);
                    acc1[r] = fmaf(xs[r * a.K + k], v, acc1[r]);
                }
        }
    }
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
        if (r < nr) {
            const float s0 = warp_sum(acc0[r]), s1 = warp_sum(acc1[r]);
            if (lane == 0) store_pair<EPI>(a, r0 + r, c0, s0, s1);
        }
    }
}

template <int EPI>
int launch_many(const GemmArgs& a, int wdt, int groups, int max_rows, cudaStream_t st) {
    dim3 grid((a.N + BN - 1) / BN, (max_rows + BM - 1) / BM, groups);
    if (wdt == 2) PGK_CUDA(launch(gemm_rows_bf16_kernel<EPI>, grid, dim3(128), 0, st, a));
    else PGK_CUDA(launch(gemm_rows_f32_kernel<EPI>, grid, dim3(128), 0, st, a));
    return 0;
}

template <typename TW, int EPI, bool ROUND>
int launch_few_t(const GemmArgs& a, int rows_per_block, cudaStream_t st, int batch) {
    const size_t smem = (size_t)rows_per_block * a.K * sizeof(float);
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        PGK_CUDA(cudaFuncSetAttribute(gemm_few_rows_kernel<TW, EPI, ROUND>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = 200 * 1024;
    }
    // a block's shared memory decides how many blocks fit an SM: keep about 16 warps per SM streaming
    const int warps = smem <= 48 * 1024 ? 4 : (smem <= 100 * 1024 ? 8 : FEW_MAX_WARPS);
    dim3 grid(((a.N + 1) / 2 + warps - 1) / warps, (a.M + rows_per_block - 1) / rows_per_block, batch);
    PGK_CUDA(launch(gemm_few_rows_kernel<TW, EPI, ROUND>, grid, dim3(warps * 32), smem, st, a, rows_per_block));
    return 0;
}

template <int EPI>
int launch_few(const GemmArgs& a, int wdt, int rows_per_block, cudaStream_t st, int batch = 1) {
    if (wdt == 2) return launch_few_t<uint16_t, EPI, true>(a, rows_per_block, st, batch);
    return launch_few_t<float, EPI, false>(a, rows_per_block, st, batch);
}

// ---------------------------------------------------------------- many rows, few columns, float32 weights (router logits)
// A 64 x 64 tile would leave all but one tile column empty and the grid a handful of blocks.  Here a warp owns SKM rows and walks
// K with a lane per element, SKN columns at a time; the partial sums meet in a warp reduction.  Plain epilogue only.
constexpr int SKM = 4, SKN = 8, SK_WARPS = 4;

__global__ void __launch_bounds__(SK_WARPS * 32) gemm_skinny_f32_kernel(GemmArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = (blockIdx.x * SK_WARPS + warp) * SKM;
    if (m0 >= a.M) return;
    const float* W = (const float*)a.W;
    for (int n0 = 0; n0 < a.N; n0 += SKN) {
        float acc[SKM][SKN];
#pragma unroll
        for (int i = 0; i < SKM; ++i)
#pragma unroll
            for (int j = 0; j < SKN; ++j) acc[i][j] = 0.f;
#pragma unroll 4
        for (int k = lane; k < a.K; k += 32) {
            float x[SKM], w[SKN];
#pragma unroll
            for (int i = 0; i < SKM; ++i) x[i] = m0 + i < a.M ? a.A[(size_t)(m0 + i) * a.lda + k] : 0.f;
#pragma unroll
            for (int j = 0; j < SKN; ++j) w[j] = n0 + j < a.N ? W[(size_t)(n0 + j) * a.K + k] : 0.f;
#pragma unroll
            for (int i = 0; i < SKM; ++i)
#pragma unroll
                for (int j = 0; j < SKN; ++j) acc[i][j] = fmaf(x[i], w[j], acc[i][j]);
        }
#pragma unroll
        for (int i = 0; i < SKM; ++i)
#pragma unroll
            for (int j = 0; j < SKN; ++j) {
                const float v = warp_sum(acc[i][j]);
                if (lane == 0 && m0 + i < a.M && n0 + j < a.N) a.C[(size_t)(m0 + i) * a.ldc + n0 + j] = v;
            }
    }
}

}  // namespace

extern "C" {

int pgk_gemm_rows_f32(const float* A, int lda, const int32_t* a_rows, const void* W, int wdt, long long w_group_stride,
                      float* C, int ldc, int M, int N, int K, const int32_t* group_off, int groups, int max_rows,
                      int epilogue, float scale, float cap, void* stream) {
    PGK_REQUIRE(wdt == 0 || wdt == 2, "gemm_rows_f32 failed: weights must be float32 (0) or bfloat16 (2), got %d", wdt);
    PGK_REQUIRE(N > 0 && K > 0 && M >= 0, "gemm_rows_f32 failed: invalid shape M=%d N=%d K=%d", M, N, K);
    PGK_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_rows_f32 failed: unknown epilogue %d", epilogue);
    PGK_REQUIRE(epilogue != 1 || N % 2 == 0, "gemm_rows_f32 failed: the gate/up epilogue needs an even N");
    const int G = group_off ? groups : 1;
    const int rows = group_off ? max_rows : M;
    if (rows <= 0 || G <= 0) return 0;
    GemmArgs a{A, a_rows, W, C, group_off, nullptr, w_group_stride, lda, ldc, M, N, K, scale, cap, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0};
    cudaStream_t st = (cudaStream_t)stream;
    if (wdt == 0 && epilogue == 0 && !group_off && !a_rows && N <= 64) {        // router logits: few columns, float32 weights
        PGK_CUDA(launch(gemm_skinny_f32_kernel, dim3((M + SK_WARPS * SKM - 1) / (SK_WARPS * SKM)), dim3(SK_WARPS * 32), 0, st, a));
        return 0;
    }
    if (epilogue == 0) return launch_many<0>(a, wdt, G, rows, st);
    if (epilogue == 1) return launch_many<1>(a, wdt, G, rows, st);
    return launch_many<2>(a, wdt, G, rows, st);
}

/* Few rows (decoding): every block of `rows_per_block` (<= 8) consecutive rows shares one weight matrix; row_group
 * (NULL: matrix 0) names it per row and must be constant inside a block. */
int pgk_gemm_few_rows_f32(const float* A, int lda, const int32_t* a_rows, const void* W, int wdt, long long w_group_stride,
                          float* C, int ldc, int M, int N, int K, const int32_t* row_group, int rows_per_block,
                          int epilogue, float scale, float cap, void* stream) {
    PGK_REQUIRE(wdt == 0 || wdt == 2, "gemm_few_rows_f32 failed: weights must be float32 (0) or bfloat16 (2), got %d", wdt);
    PGK_REQUIRE(N > 0 && K > 0 && M >= 0, "gemm_few_rows_f32 failed: invalid shape M=%d N=%d K=%d", M, N, K);
    PGK_REQUIRE(rows_per_block >= 1 && rows_per_block <= RMAX, "gemm_few_rows_f32 failed: 1..%d rows per block", RMAX);
    PGK_REQUIRE((size_t)rows_per_block * K * 4 <= 200 * 1024, "gemm_few_rows_f32 failed: %d rows of K=%d do not fit shared memory", rows_per_block, K);
    PGK_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_few_rows_f32 failed: unknown epilogue %d", epilogue);
    PGK_REQUIRE(epilogue != 1 || N % 2 == 0, "gemm_few_rows_f32 failed: the gate/up epilogue needs an even N");
    if (M == 0) return 0;
    GemmArgs a{A, a_rows, W, C, nullptr, row_group, w_group_stride, lda, ldc, M, N, K, scale, cap, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0};
    cudaStream_t st = (cudaStream_t)stream;
    if (epilogue == 0) return launch_few<0>(a, wdt, rows_per_block, st);
    if (epilogue == 1) return launch_few<1>(a, wdt, rows_per_block, st);
    return launch_few<2>(a, wdt, rows_per_block, st);
}


/* The general form: `batch` independent products (A columns a_batch apart, matrices w_batch apart, C columns c_batch apart)
 * over the same M rows, every epilogue.  rows_per_block > 0 selects the few-row kernel (M <= 8 rows share one pass over the
 * weights), 0 the tiled kernel. */
int pgk_gemm_seq_f32(const float* A, int lda, long long a_batch, const void* W, int wdt, long long w_batch, float* C, int ldc,
                     long long c_batch, int M, int N, int K, int batch, int epilogue, float p0, float p1, const float* col_scale,
                     const void* aux, int aux_dtype, const int32_t* aux_rows, int aux_ld, int aux_off, int rows_per_block,
                     void* stream) {
    PGK_REQUIRE(wdt == 0 || wdt == 2, "gemm_seq_f32 failed: weights must be float32 (0) or bfloat16 (2), got %d", wdt);
    PGK_REQUIRE(N > 0 && K > 0 && M >= 0 && batch >= 1, "gemm_seq_f32 failed: invalid shape M=%d N=%d K=%d batch=%d", M, N, K, batch);
    PGK_REQUIRE(epilogue >= 0 && epilogue <= 6, "gemm_seq_f32 failed: unknown epilogue %d", epilogue);
    PGK_REQUIRE((epilogue != 1 && epilogue != 3) || N % 2 == 0, "gemm_seq_f32 failed: a gate/up epilogue needs an even N");
    PGK_REQUIRE(epilogue != 4 || col_scale, "gemm_seq_f32 failed: the scaled-accumulate epilogue needs its column factors");
    PGK_REQUIRE(epilogue != 5 || (aux && aux_rows && (aux_dtype == 0 || aux_dtype == 2)), "gemm_seq_f32 failed: the gather epilogue needs its table and rows");
    PGK_REQUIRE(rows_per_block >= 0 && rows_per_block <= RMAX, "gemm_seq_f32 failed: 0..%d rows per block", RMAX);
    PGK_REQUIRE(rows_per_block == 0 || (size_t)rows_per_block * K * 4 <= 200 * 1024, "gemm_seq_f32 failed: %d rows of K=%d do not fit shared memory", rows_per_block, K);
    if (M == 0) return 0;
    GemmArgs a{A, nullptr, W, C, nullptr, nullptr, w_batch, lda, ldc, M, N, K, p0, p1, col_scale, aux, aux_rows, aux_ld, aux_off, aux_dtype, a_batch, c_batch};
    cudaStream_t st = (cudaStream_t)stream;
    if (rows_per_block > 0) {
        switch (epilogue) {
            case 0: return launch_few<0>(a, wdt, rows_per_block, st, batch);
            case 1: return launch_few<1>(a, wdt, rows_per_block, st, batch);
            case 2: return launch_few<2>(a, wdt, rows_per_block, st, batch);
            case 3: return launch_few<3>(a, wdt, rows_per_block, st, batch);
            case 4: return launch_few<4>(a, wdt, rows_per_block, st, batch);
            case 5: return launch_few<5>(a, wdt, rows_per_block, st, batch);
            default: return launch_few<6>(a, wdt, rows_per_block, st, batch);
        }
    }
    switch (epilogue) {
        case 0: return launch_many<0>(a, wdt, batch, M, st);
        case 1: return launch_many<1>(a, wdt, batch, M, st);
        case 2: return launch_many<2>(a, wdt, batch, M, st);
        case 3: return launch_many<3>(a, wdt, batch, M, st);
        case 4: return launch_many<4>(a, wdt, batch, M, st);
        case 5: return launch_many<5>(a, wdt, batch, M, st);
        default: return launch_many<6>(a, wdt, batch, M, st);
    }
}

}  // extern "C"
