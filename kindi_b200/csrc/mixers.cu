// Kernels of mixers beside plain attention: an output gate, a gated RMS norm over the concatenated heads, the steps
// of latent attention around its products (norms of the latents, rotation of interleaved pairs, the store of the
// latent into the cache, per-head products), and the decayed outer-product recurrence of linear attention.
// Storage is float or bf16, all arithmetic 32-bit; every sum has an order that depends on sizes and positions only,
// so a row's result does not depend on the batch or on how a prompt was cut into steps.
#include "common.cuh"

// element i of a row that came either as a row or as 32-bit planes whose sum (in order) it is
template <typename TIN>
__device__ __forceinline__ float mx_rd(const TIN* src, int n_planes, size_t plane_stride, size_t i) {
    float v = kb_to_f<TIN>(src[i]);
    for (int s = 1; s < n_planes; s++) v += kb_to_f<TIN>(src[(size_t)s * plane_stride + i]);
    return v;
}
__device__ __forceinline__ float mx_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float mx_silu(float z) { return z / (1.0f + expf(-z)); }
// (the fast exponential and division: their error is far below one bf16 rounding; the serving path's long prompts)
__device__ __forceinline__ float mx_silu_fast(float z) { return __fdividef(z, 1.0f + __expf(-z)); }

// sum over the block's threads in a fixed order (lanes by butterfly, warps in warp order); every thread gets it
__device__ __forceinline__ float mx_block_sum(float v, float* red) {
    v = kb_warp_sum(v);
    __syncthreads();                                  // (red may still be read from the call before)
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.0f;
    for (int k = 0; k < (int)(blockDim.x >> 5); k++) tot += red[k];
    return tot;
}

// ------------------------------------------------------------------------------------------------ output gate
// out[t][c] = a[t][c] * sigmoid(g[t][c]); g rows or planes
template <typename TA, typename TG>
__global__ void __launch_bounds__(256) k_gate_mul(const TA* KB_STEP_DATA a, int lda, const TG* KB_STEP_DATA g,
        int n_planes, size_t plane_stride, int ldg, TA* out, int ldo, int N) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int c = blockIdx.y * 256 + threadIdx.x;
    if (c >= N) return;
    const size_t t = blockIdx.x;
    const float z = mx_rd<TG>(g + t * ldg, n_planes, plane_stride, c);
    out[t * ldo + c] = kb_from_f<TA>(kb_to_f<TA>(a[t * lda + c]) * mx_sigmoid(z));
}

extern "C" int kb_gate_mul(const void* a, int adtype, int lda, const void* g, int gdtype, int n_planes,
                           long long plane_stride, int ldg, void* out, int ldo, int T, int N, cudaStream_t st) {
    if (T <= 0 || N <= 0) return 0;
    dim3 grid(T, (N + 255) / 256);
    if (adtype == KB_F32 && gdtype == KB_F32)
        kb_launch(k_gate_mul<float, float>, grid, 256, 0, st, (const float*)a, lda, (const float*)g, n_planes,
                  (size_t)plane_stride, ldg, (float*)out, ldo, N);
    else if (adtype == KB_BF16 && gdtype == KB_BF16)
        kb_launch(k_gate_mul<bf16, bf16>, grid, 256, 0, st, (const bf16*)a, lda, (const bf16*)g, n_planes,
                  (size_t)plane_stride, ldg, (bf16*)out, ldo, N);
    else if (adtype == KB_BF16 && gdtype == KB_F32)
        kb_launch(k_gate_mul<bf16, float>, grid, 256, 0, st, (const bf16*)a, lda, (const float*)g, n_planes,
                  (size_t)plane_stride, ldg, (bf16*)out, ldo, N);
    else return (int)cudaErrorInvalidValue;
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ gated RMS norm
// out[t][c] = x[t][c] / sqrt(mean_c(x[t]^2) + eps) * w[c] * sigmoid(g[t][c]): the heads' 32-bit outputs normalised
// together, gated, and written in the run's type for the output product. One block per row.
template <typename TG, typename TW, typename TO>
__global__ void __launch_bounds__(256) k_gated_rmsnorm(const float* KB_STEP_DATA x, int ldx, const TW* __restrict__ w,
        float eps, const TG* KB_STEP_DATA g, int n_planes, size_t plane_stride, int ldg, TO* __restrict__ out, int ldo,
        int N) {
    __shared__ float red[8];
    kb_pdl_launch();
    kb_pdl_wait();
    const size_t t = blockIdx.x;
    const float* xr = x + t * ldx;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < N; c += 256) ss = fmaf(xr[c], xr[c], ss);
    const float tot = mx_block_sum(ss, red);
    const float scale = 1.0f / sqrtf(tot / (float)N + eps);
    for (int c = threadIdx.x; c < N; c += 256) {
        const float y = __fmul_rn(__fmul_rn(scale, xr[c]), kb_to_f<TW>(w[c]));
        float z = 1.0f;
        if (g != nullptr) z = mx_sigmoid(mx_rd<TG>(g + t * ldg, n_planes, plane_stride, c));
        out[t * ldo + c] = kb_from_f<TO>(y * z);
    }
}

extern "C" int kb_gated_rmsnorm(const float* x, int ldx, const void* w, int wdtype, float eps, const void* g,
                                int gdtype, int n_planes, long long plane_stride, int ldg, void* out, int odtype,
                                int ldo, int T, int N, cudaStream_t st) {
    if (T <= 0 || N <= 0) return 0;
#define KB_GN(TG, TW, TO)                                                                                        \
    kb_launch(k_gated_rmsnorm<TG, TW, TO>, T, 256, 0, st, x, ldx, (const TW*)w, eps, (const TG*)g, n_planes,     \
              (size_t)plane_stride, ldg, (TO*)out, ldo, N)
    if (odtype == KB_F32 && wdtype == KB_F32 && gdtype == KB_F32) KB_GN(float, float, float);
    else if (odtype == KB_BF16 && wdtype == KB_BF16 && gdtype == KB_BF16) KB_GN(bf16, bf16, bf16);
    else if (odtype == KB_BF16 && wdtype == KB_BF16 && gdtype == KB_F32) KB_GN(float, bf16, bf16);
    else if (odtype == KB_BF16 && wdtype == KB_F32 && gdtype == KB_BF16) KB_GN(bf16, float, bf16);
    else if (odtype == KB_BF16 && wdtype == KB_F32 && gdtype == KB_F32) KB_GN(float, float, bf16);
    else return (int)cudaErrorInvalidValue;
#undef KB_GN
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ latent attention
// The down projections of a row come as [query latent (q_rank) | key/value latent (kv_rank) | rotated key part (rot)
// | anything else], as a row or as planes. This kernel writes the normalised query latent (RMS norm with gains, the
// run's type) and stores into the cache, at the row's position, ONE key/value head of size D >= kv_rank + rot:
//   keys   [normalised latent | rotated part | zeros]      values [normalised latent | zeros]
// so that attention over the cache with queries [W_uk^T q | rotated q | zeros] gives the scores of the expanded keys,
// and its output's first kv_rank elements are the weighted sum of latents, from which W_uv makes the heads' values.
// Rotation: element 2i pairs with 2i + 1; angle = (float)pos * freq[i]; cosine and sine are multiplied by mult.
template <typename TIN, typename TW, typename T>
__global__ void __launch_bounds__(256) k_latent_prep(const TIN* KB_STEP_DATA in, int n_planes, size_t plane_stride,
        int ld_in, int q_rank, int kv_rank, int rot, const TW* __restrict__ wq, const TW* __restrict__ wkv, float eps,
        const float* __restrict__ freq, float mult, const int* __restrict__ pos, const int* __restrict__ seq,
        const int* __restrict__ slot, T* __restrict__ cq, int ldcq, KbCacheView cv, int* status) {
    __shared__ float red[8];
    kb_pdl_launch();
    const int t = blockIdx.x;
    const int p = pos[t];
    T* cqr = cq + (size_t)t * ldcq;
    kb_pdl_wait();
    if (p < 0) {                                       // a padding row of a recorded step: a defined query latent, no store
        for (int i = threadIdx.x; i < q_rank; i += 256) cqr[i] = kb_from_f<T>(0.0f);
        return;
    }
    const TIN* src = in + (size_t)t * ld_in;
    float sq = 0.0f, sc = 0.0f;
    for (int i = threadIdx.x; i < q_rank; i += 256) {
        const float v = mx_rd<TIN>(src, n_planes, plane_stride, i);
        sq = fmaf(v, v, sq);
    }
    for (int i = threadIdx.x; i < kv_rank; i += 256) {
        const float v = mx_rd<TIN>(src, n_planes, plane_stride, q_rank + i);
        sc = fmaf(v, v, sc);
    }
    const float tq = mx_block_sum(sq, red);
    const float tc = mx_block_sum(sc, red);
    const float scale_q = 1.0f / sqrtf(tq / (float)q_rank + eps);
    const float scale_c = 1.0f / sqrtf(tc / (float)kv_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += 256)
        cqr[i] = kb_from_f<T>(__fmul_rn(__fmul_rn(scale_q, mx_rd<TIN>(src, n_planes, plane_stride, i)), kb_to_f<TW>(wq[i])));
    const int s = slot[seq[t]];
    const int page = cv.table[(size_t)s * cv.table_stride + p / KB_PAGE];
    if (page < 0 || page >= cv.n_pages) {
        if (threadIdx.x == 0) atomicOr(status, KB_ST_BAD_PAGE);
        return;
    }
    T* kd = (T*)cv.pool + kb_kv_offset(cv, page, 0, 0, p % KB_PAGE);
    T* vd = (T*)cv.pool + kb_kv_offset(cv, page, 1, 0, p % KB_PAGE);
    for (int i = threadIdx.x; i < kv_rank; i += 256) {
        const T c = kb_from_f<T>(__fmul_rn(__fmul_rn(scale_c, mx_rd<TIN>(src, n_planes, plane_stride, q_rank + i)),
                                           kb_to_f<TW>(wkv[i])));
        kd[i] = c;
        vd[i] = c;
    }
    for (int i = threadIdx.x; i < rot / 2; i += 256) {
        const float ang = __fmul_rn((float)p, freq[i]);
        const float c = __fmul_rn(cosf(ang), mult), sn = __fmul_rn(sinf(ang), mult);
        const float a = mx_rd<TIN>(src, n_planes, plane_stride, q_rank + kv_rank + 2 * i);
        const float b = mx_rd<TIN>(src, n_planes, plane_stride, q_rank + kv_rank + 2 * i + 1);
        kd[kv_rank + 2 * i] = kb_from_f<T>(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn)));
        kd[kv_rank + 2 * i + 1] = kb_from_f<T>(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn)));
    }
    for (int i = kv_rank + rot + threadIdx.x; i < cv.head_dim; i += 256) kd[i] = kb_from_f<T>(0.0f);
    for (int i = kv_rank + threadIdx.x; i < cv.head_dim; i += 256) vd[i] = kb_from_f<T>(0.0f);
}

extern "C" int kb_latent_prep(const void* in, int in_dtype, int n_planes, long long plane_stride, int ld_in, int q_rank,
                              int kv_rank, int rot, const void* wq, const void* wkv, int wdtype, float eps,
                              const float* freq, float mult, const int* pos, const int* seq, const int* slot, void* cq,
                              int dtype, int ldcq, int T, int D, void* pool, const int* table, int table_stride,
                              int n_pages, int* status, cudaStream_t st) {
    if (T <= 0) return 0;
    if (rot % 2 || kv_rank + rot > D) return (int)cudaErrorInvalidValue;
    KbCacheView cv{pool, table, table_stride, n_pages, 1, D};
#define KB_LP(TIN, TW, T_)                                                                                       \
    kb_launch(k_latent_prep<TIN, TW, T_>, T, 256, 0, st, (const TIN*)in, n_planes, (size_t)plane_stride, ld_in,  \
              q_rank, kv_rank, rot, (const TW*)wq, (const TW*)wkv, eps, freq, mult, pos, seq, slot, (T_*)cq, ldcq, \
              cv, status)
    if (in_dtype == KB_F32 && dtype == KB_F32 && wdtype == KB_F32) KB_LP(float, float, float);
    else if (in_dtype == KB_F32 && dtype == KB_BF16 && wdtype == KB_BF16) KB_LP(float, bf16, bf16);
    else if (in_dtype == KB_BF16 && dtype == KB_BF16 && wdtype == KB_BF16) KB_LP(bf16, bf16, bf16);
    else if (in_dtype == KB_F32 && dtype == KB_BF16 && wdtype == KB_F32) KB_LP(float, float, bf16);
    else if (in_dtype == KB_BF16 && dtype == KB_BF16 && wdtype == KB_F32) KB_LP(bf16, float, bf16);
    else return (int)cudaErrorInvalidValue;
#undef KB_LP
    KB_LAUNCH_RET();
}

// The rotated part of every query head: q[t][h] = [plain (dim) | rotated (rot)] -> out[t][h][at .. at + rot) rotated
// (interleaved pairs), out[t][h][at + rot .. D) = 0. The first `at` elements of each head are written by the per-head
// product below.
template <typename T>
__global__ void k_latent_qrope(const T* KB_STEP_DATA q, int ldq, int dim, int rot, const float* __restrict__ freq,
        float mult, const int* __restrict__ pos, T* __restrict__ out, int ldo, int at, int D) {
    kb_pdl_launch();
    const int t = blockIdx.x, h = blockIdx.y;
    const int p = pos[t];
    kb_pdl_wait();
    const T* src = q + (size_t)t * ldq + (size_t)h * (dim + rot) + dim;
    T* dst = out + (size_t)t * ldo + (size_t)h * D + at;
    if (p >= 0) {
        for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) {
            const float ang = __fmul_rn((float)p, freq[i]);
            const float c = __fmul_rn(cosf(ang), mult), sn = __fmul_rn(sinf(ang), mult);
            const float a = kb_to_f<T>(src[2 * i]), b = kb_to_f<T>(src[2 * i + 1]);
            dst[2 * i] = kb_from_f<T>(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn)));
            dst[2 * i + 1] = kb_from_f<T>(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn)));
        }
    } else {
        for (int i = threadIdx.x; i < rot; i += blockDim.x) dst[i] = kb_from_f<T>(0.0f);
    }
    for (int i = rot + threadIdx.x; i < D - at; i += blockDim.x) dst[i] = kb_from_f<T>(0.0f);
}

extern "C" int kb_latent_qrope(const void* q, int dtype, int ldq, int dim, int rot, const float* freq, float mult,
                               const int* pos, void* out, int ldo, int at, int D, int T, int H, cudaStream_t st) {
    if (T <= 0 || H <= 0) return 0;
    if (rot % 2 || at + rot > D) return (int)cudaErrorInvalidValue;
    dim3 grid(T, H);
    if (dtype == KB_F32)
        kb_launch(k_latent_qrope<float>, grid, 64, 0, st, (const float*)q, ldq, dim, rot, freq, mult, pos, (float*)out,
                  ldo, at, D);
    else
        kb_launch(k_latent_qrope<bf16>, grid, 64, 0, st, (const bf16*)q, ldq, dim, rot, freq, mult, pos, (bf16*)out,
                  ldo, at, D);
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ per-head products
// out[t][h * ldoh + n] = sum_k a[t][h * ldah + k] * w[h][n][k] (n < N, k < K; w [H][N][K] contiguous), every sum over
// k = 0, 1, 2, ... in order with 32-bit fused multiply-adds. With gate: out *= sigmoid(gate[t][h * N + n]) (rows or
// planes). grid.z = head.
#define HG_BM 64
#define HG_BN 64
#define HG_BK 32
template <typename TA, typename TW, typename TG>
__global__ void __launch_bounds__(256) k_head_gemm(const TA* KB_STEP_DATA A, int lda, int ldah, const TW* __restrict__ W,
        TA* __restrict__ C, int ldc, int ldch, int M, int N, int K, const TG* KB_STEP_DATA gate, int n_planes,
        size_t plane_stride, int ldg) {
    __shared__ float As[HG_BK][HG_BM + 1];
    __shared__ float Ws[HG_BK][HG_BN + 1];
    kb_pdl_launch();
    kb_pdl_wait();
    const int h = blockIdx.z;
    const int m0 = blockIdx.y * HG_BM, n0 = blockIdx.x * HG_BN;
    const TA* Ah = A + (size_t)h * ldah;
    const TW* Wh = W + (size_t)h * N * K;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    constexpr int PER = HG_BM * HG_BK / 256;
    for (int k0 = 0; k0 < K; k0 += HG_BK) {
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const int e = tid + 256 * j, r = e / HG_BK, c = e % HG_BK;
            const int m = m0 + r, n = n0 + r, k = k0 + c;
            As[c][r] = (m < M && k < K) ? kb_to_f<TA>(Ah[(size_t)m * lda + k]) : 0.0f;
            Ws[c][r] = (n < N && k < K) ? kb_to_f<TW>(Wh[(size_t)n * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HG_BK; k++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (gate != nullptr)
                v *= mx_sigmoid(mx_rd<TG>(gate + (size_t)m * ldg, n_planes, plane_stride, (size_t)h * N + n));
            C[(size_t)m * ldc + (size_t)h * ldch + n] = kb_from_f<TA>(v);
        }
    }
}

// The same products for bf16 operands on the tensor cores (mma.sync m16n8k16, 32-bit accumulators): a block of four
// warps takes 64 rows x 64 columns of one head, a warp 16 rows x 64 columns; K runs in blocks of 32 through shared
// memory (rows padded to 40 elements: the fragment loads meet no bank conflicts). Needs K % 8 == 0 and 16-byte
// aligned rows of A and W (the loads are 16 bytes wide); a sum's order depends on K only.
__device__ __forceinline__ void mx_mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
#define HM_BM 64
#define HM_BN 64
#define HM_BK 32
#define HM_LD 40
template <typename TG>
__global__ void __launch_bounds__(128) k_head_gemm_mma(const bf16* KB_STEP_DATA A, int lda, int ldah,
        const bf16* __restrict__ W, bf16* __restrict__ C, int ldc, int ldch, int M, int N, int K,
        const TG* KB_STEP_DATA gate, int n_planes, size_t plane_stride, int ldg) {
    __shared__ __align__(16) bf16 As[HM_BM * HM_LD];
    __shared__ __align__(16) bf16 Ws[HM_BN * HM_LD];
    kb_pdl_launch();
    const int h = blockIdx.z;
    const int m0 = blockIdx.y * HM_BM, n0 = blockIdx.x * HM_BN;
    const bf16* Ah = A + (size_t)h * ldah;
    const bf16* Wh = W + (size_t)h * N * K;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[j][i] = 0.0f;
    const int lr = tid >> 2, lc = (tid & 3) * 8;       // this thread's rows (lr, lr + 32) and 8-element piece of a K block
    kb_pdl_wait();
    for (int k0 = 0; k0 < K; k0 += HM_BK) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int r = lr + 32 * half, k = k0 + lc;
            uint4 av = make_uint4(0u, 0u, 0u, 0u), wv = make_uint4(0u, 0u, 0u, 0u);
            if (m0 + r < M && k < K) av = *(const uint4*)(Ah + (size_t)(m0 + r) * lda + k);
            if (n0 + r < N && k < K) wv = *(const uint4*)(Wh + (size_t)(n0 + r) * K + k);
            *(uint4*)(As + r * HM_LD + lc) = av;
            *(uint4*)(Ws + r * HM_LD + lc) = wv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HM_BK; kk += 16) {
            uint32_t a[4];
            const bf16* ar = As + (warp * 16 + g) * HM_LD + kk + 2 * t;
            a[0] = *(const uint32_t*)(ar);
            a[1] = *(const uint32_t*)(ar + 8 * HM_LD);
            a[2] = *(const uint32_t*)(ar + 8);
            a[3] = *(const uint32_t*)(ar + 8 * HM_LD + 8);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const bf16* wr = Ws + (j * 8 + g) * HM_LD + kk + 2 * t;
                mx_mma_bf16(acc[j], a, *(const uint32_t*)(wr), *(const uint32_t*)(wr + 8));
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int m = m0 + warp * 16 + g + (i >> 1) * 8, n = n0 + j * 8 + 2 * t + (i & 1);
            if (m >= M || n >= N) continue;
            float v = acc[j][i];
            if (gate != nullptr)
                v *= mx_sigmoid(mx_rd<TG>(gate + (size_t)m * ldg, n_planes, plane_stride, (size_t)h * N + n));
            C[(size_t)m * ldc + (size_t)h * ldch + n] = __float2bfloat16_rn(v);
        }
}

extern "C" int kb_head_gemm(const void* A, int adtype, int lda, int ldah, const void* W, int wdtype, void* C, int ldc,
                            int ldch, int M, int N, int K, int H, const void* gate, int gdtype, int n_planes,
                            long long plane_stride, int ldg, cudaStream_t st, int tensor_cores) {
    if (M <= 0 || N <= 0 || H <= 0) return 0;
    if (H > 65535) return (int)cudaErrorInvalidValue;
    if (tensor_cores && adtype == KB_BF16 && wdtype == KB_BF16 && K % 8 == 0 && lda % 8 == 0 && ldah % 8 == 0 &&
        ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0) {
        dim3 gm((N + HM_BN - 1) / HM_BN, (M + HM_BM - 1) / HM_BM, H);
        if (gate == nullptr || gdtype == KB_F32)
            kb_launch(k_head_gemm_mma<float>, gm, 128, 0, st, (const bf16*)A, lda, ldah, (const bf16*)W, (bf16*)C, ldc,
                      ldch, M, N, K, (const float*)gate, n_planes, (size_t)plane_stride, ldg);
        else
            kb_launch(k_head_gemm_mma<bf16>, gm, 128, 0, st, (const bf16*)A, lda, ldah, (const bf16*)W, (bf16*)C, ldc,
                      ldch, M, N, K, (const bf16*)gate, n_planes, (size_t)plane_stride, ldg);
        KB_LAUNCH_RET();
    }
    dim3 grid((N + HG_BN - 1) / HG_BN, (M + HG_BM - 1) / HG_BM, H);
#define KB_HG(TA, TW, TG)                                                                                       \
    kb_launch(k_head_gemm<TA, TW, TG>, grid, 256, 0, st, (const TA*)A, lda, ldah, (const TW*)W, (TA*)C, ldc,    \
              ldch, M, N, K, (const TG*)gate, n_planes, (size_t)plane_stride, ldg)
    const bool gf = gate == nullptr || gdtype == KB_F32;
    if (adtype == KB_F32 && wdtype == KB_F32 && gf) KB_HG(float, float, float);
    else if (adtype == KB_BF16 && wdtype == KB_BF16 && gf) KB_HG(bf16, bf16, float);
    else if (adtype == KB_BF16 && wdtype == KB_BF16) KB_HG(bf16, bf16, bf16);
    else if (adtype == KB_BF16 && wdtype == KB_F32 && gf) KB_HG(bf16, float, float);
    else if (adtype == KB_BF16 && wdtype == KB_F32) KB_HG(bf16, float, bf16);
    else return (int)cudaErrorInvalidValue;
#undef KB_HG
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ decayed recurrence
// Linear attention with a decay per head. The projections of a row come as [q (H x d) | k (H x d) | v (H x dv) | ...]
// (a row or planes); q, k and v pass through silu. Per sequence and head the state S (d x dv, 32-bit, kept per cache
// slot as [H][dv][d]) follows S <- decay * S + k v^T token by token, and the row's output is o = S^T q (32-bit,
// [T][H * dv]). The columns of S are independent recurrences: a warp owns one column (its d elements spread over the
// lanes), a block eight columns of one (sequence, head); the block stages the q, k and v of a run of tokens in shared
// memory. Sequences are taken by their row ranges (q_start), so padding rows are never touched; a sequence's state
// is read at the start of its rows and written back after them, whatever their number.
#define DS_COLS 8
#define DS_CHUNK 16
#define DS_MAX_DPL 8            // d up to 256
template <typename TIN>
__global__ void __launch_bounds__(32 * DS_COLS) k_decay_scan(const TIN* KB_STEP_DATA in, int n_planes, size_t plane_stride,
        int ld_in, int H, int d, int dv, const float* __restrict__ decay, const int* __restrict__ q_start,
        const int* __restrict__ slot, float* state, float* __restrict__ out, int ldo) {
    extern __shared__ float sm[];
    float* qs = sm;                                   // [DS_CHUNK][d]
    float* ks = qs + DS_CHUNK * d;                    // [DS_CHUNK][d]
    float* vs = ks + DS_CHUNK * d;                    // [DS_CHUNK][DS_COLS]
    kb_pdl_launch();
    const int b = blockIdx.x / H, h = blockIdx.x % H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e0 = blockIdx.y * DS_COLS, e = e0 + warp;
    const int r0 = q_start[b], r1 = q_start[b + 1];
    const float lam = decay[h];
    float* srow = state + (((size_t)slot[b] * H + h) * dv + (e < dv ? e : 0)) * d;
    kb_pdl_wait();
    float S[DS_MAX_DPL];
#pragma unroll
    for (int i = 0; i < DS_MAX_DPL; i++) {
        const int j = lane + 32 * i;
        S[i] = (e < dv && j < d) ? srow[j] : 0.0f;
    }
    const size_t oq = (size_t)h * d, ok = (size_t)H * d + (size_t)h * d, ov = (size_t)2 * H * d + (size_t)h * dv;
    for (int c0 = r0; c0 < r1; c0 += DS_CHUNK) {
        const int n = min(DS_CHUNK, r1 - c0);
        for (int idx = threadIdx.x; idx < n * d; idx += 32 * DS_COLS) {
            const int t = idx / d, j = idx % d;
            const TIN* src = in + (size_t)(c0 + t) * ld_in;
            qs[t * d + j] = mx_silu(mx_rd<TIN>(src, n_planes, plane_stride, oq + j));
            ks[t * d + j] = mx_silu(mx_rd<TIN>(src, n_planes, plane_stride, ok + j));
        }
        for (int idx = threadIdx.x; idx < n * DS_COLS; idx += 32 * DS_COLS) {
            const int t = idx / DS_COLS, w = idx % DS_COLS;
            const TIN* src = in + (size_t)(c0 + t) * ld_in;
            vs[idx] = (e0 + w < dv) ? mx_silu(mx_rd<TIN>(src, n_planes, plane_stride, ov + e0 + w)) : 0.0f;
        }
        __syncthreads();
        for (int t = 0; t < n; t++) {
            const float vt = vs[t * DS_COLS + warp];
            float p = 0.0f;
#pragma unroll
            for (int i = 0; i < DS_MAX_DPL; i++) {
                const int j = lane + 32 * i;
                if (j < d) {
                    S[i] = fmaf(lam, S[i], __fmul_rn(ks[t * d + j], vt));
                    p = fmaf(S[i], qs[t * d + j], p);
                }
            }
            p = kb_warp_sum(p);
            if (lane == 0 && e < dv) out[(size_t)(c0 + t) * ldo + (size_t)h * dv + e] = p;
        }
        __syncthreads();
    }
    if (e < dv && r1 > r0) {
#pragma unroll
        for (int i = 0; i < DS_MAX_DPL; i++) {
            const int j = lane + 32 * i;
            if (j < d) srow[j] = S[i];
        }
    }
}

// The same recurrence for long prompts, parallel over runs ("chunks") of C tokens. The recurrence is linear in the
// state, so a sequence's chunks can be worked on side by side:
//   1. every chunk but the last: its own contribution P_c = sum_j decay^(C - 1 - j) k_j v_j^T from a zero state
//      (k_decay_chunk<.., false, ..>; the blocks of chunk 0 also keep a copy of the state the sequence came with);
//   2. element by element over the chunks: S_c = decay^C S_(c-1) + P_c, leaving in P[c] the state BEFORE chunk c
//      (k_decay_prefix);
//   3. every chunk: from the state before it, the token-by-token recurrence over its own rows with the outputs;
//      the last chunk's blocks store the sequence's new state (k_decay_chunk<.., true, ..>).
// A warp owns DC_CW columns of the state (four independent sums in flight), a block 32 columns; the next tile of
// tokens is fetched into registers while the current one is worked on. All arithmetic is 32-bit; the sums differ
// from the token-by-token kernel's by rounding only (decay^C is taken by powf, silu by the fast exponential).
#define DC_CW 4
#define DC_COLS (8 * DC_CW)
#define DC_TILE 16
#define DC_PER_V (DC_TILE * DC_COLS / 256)
// DPL = elements of a column a lane holds: ceil(d / 32) rounded up to 1, 2, 4 or 8
template <typename TIN, bool OUT, int DPL>
__global__ void __launch_bounds__(256) k_decay_chunk(const TIN* KB_STEP_DATA in, int n_planes, size_t plane_stride,
        int ld_in, int H, int d, int dv, const float* __restrict__ decay, const int* __restrict__ q_start,
        const int* __restrict__ slot, float* state, float* P, float* S0, float* __restrict__ out, int ldo, int C,
        int nc_max) {
    extern __shared__ float sm[];
    float* qs = sm;                                   // [DC_TILE][32 DPL]
    float* ks = qs + DC_TILE * 32 * DPL;              // [DC_TILE][32 DPL] (rows of the power-of-two length, zeros past d)
    float* vs = ks + DC_TILE * 32 * DPL;              // [DC_TILE][DC_COLS]
    constexpr int DR = 32 * DPL;                       // a staged row's length: d rounded up to a power of two
    constexpr int DC_PER_QK = DC_TILE * DR / 256;
    kb_pdl_launch();
    const int b = blockIdx.x / H, h = blockIdx.x % H, c = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e0 = blockIdx.y * DC_COLS, ew = e0 + warp * DC_CW;
    const int r0 = q_start[b], r1 = q_start[b + 1];
    const int nc = (r1 - r0 + C - 1) / C;
    if (c >= nc) return;
    const bool last = c == nc - 1;
    const float lam = decay[h];
    const size_t bh = (size_t)b * H + h;
    float* srow = state + ((size_t)slot[b] * H + h) * dv * d;
    float* s0row = S0 + bh * dv * d;
    kb_pdl_wait();
    float S[DC_CW][DPL];
    if (!OUT) {
        if (c == 0) {
            // the state the sequence came with, for the blocks of the second pass (which overwrite the slot's own)
            for (int x = 0; x < DC_CW; x++)
#pragma unroll
                for (int i = 0; i < DPL; i++) {
                    const int j = lane + 32 * i;
                    if (ew + x < dv && j < d) s0row[(size_t)(ew + x) * d + j] = srow[(size_t)(ew + x) * d + j];
                }
        }
        if (last) return;
#pragma unroll
        for (int x = 0; x < DC_CW; x++)
#pragma unroll
            for (int i = 0; i < DPL; i++) S[x][i] = 0.0f;
    } else {
        // the state before this chunk, as the scan kernel left it in P[c]
        const float* pr = P + (bh * nc_max + c) * dv * d;
#pragma unroll
        for (int x = 0; x < DC_CW; x++)
#pragma unroll
            for (int i = 0; i < DPL; i++) {
                const int j = lane + 32 * i;
                S[x][i] = (ew + x < dv && j < d) ? pr[(size_t)(ew + x) * d + j] : 0.0f;
            }
    }
    const int ra = r0 + c * C, rz = min(ra + C, r1);
    const size_t oq = (size_t)h * d, ok = (size_t)H * d + (size_t)h * d, ov = (size_t)2 * H * d + (size_t)h * dv;
    float rq[DC_PER_QK], rk[DC_PER_QK], rv[DC_PER_V];
    auto fetch = [&](int t0) {
        const int n = min(DC_TILE, rz - t0);
#pragma unroll
        for (int u = 0; u < DC_PER_QK; u++) {
            const int idx = threadIdx.x + 256 * u;
            const int t = idx / DR, j = idx % DR;
            rq[u] = rk[u] = 0.0f;
            if (t < n && j < d) {
                const TIN* src = in + (size_t)(t0 + t) * ld_in;
                if (OUT) rq[u] = mx_silu_fast(mx_rd<TIN>(src, n_planes, plane_stride, oq + j));
                rk[u] = mx_silu_fast(mx_rd<TIN>(src, n_planes, plane_stride, ok + j));
            }
        }
#pragma unroll
        for (int u = 0; u < DC_PER_V; u++) {
            const int idx = threadIdx.x + 256 * u;
            const int t = idx / DC_COLS, w = idx % DC_COLS;
            rv[u] = 0.0f;
            if (t < n && e0 + w < dv)
                rv[u] = mx_silu_fast(mx_rd<TIN>(in + (size_t)(t0 + t) * ld_in, n_planes, plane_stride, ov + e0 + w));
        }
    };
    auto stage = [&](int t0) {
#pragma unroll
        for (int u = 0; u < DC_PER_QK; u++) {
            const int idx = threadIdx.x + 256 * u;
            if (OUT) qs[idx] = rq[u];
            ks[idx] = rk[u];
        }
#pragma unroll
        for (int u = 0; u < DC_PER_V; u++) vs[threadIdx.x + 256 * u] = rv[u];
    };
    fetch(ra);
    for (int t0 = ra; t0 < rz; t0 += DC_TILE) {
        stage(t0);
        __syncthreads();
        if (t0 + DC_TILE < rz) fetch(t0 + DC_TILE);
        const int n = min(DC_TILE, rz - t0);
        for (int t = 0; t < n; t++) {
            float kk[DPL], qq[DPL], pp[DC_CW];
#pragma unroll
            for (int i = 0; i < DPL; i++) {
                const int j = lane + 32 * i;
                kk[i] = ks[t * DR + j];
                qq[i] = OUT ? qs[t * DR + j] : 0.0f;
            }
#pragma unroll
            for (int x = 0; x < DC_CW; x++) {
                const float vt = vs[t * DC_COLS + warp * DC_CW + x];
                float p = 0.0f;
#pragma unroll
                for (int i = 0; i < DPL; i++) {
                    if (lane + 32 * i < d) {
                        S[x][i] = fmaf(lam, S[x][i], __fmul_rn(kk[i], vt));
                        if (OUT) p = fmaf(S[x][i], qq[i], p);
                    }
                }
                pp[x] = p;
            }
            if (OUT) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                    for (int x = 0; x < DC_CW; x++) pp[x] += __shfl_xor_sync(0xffffffffu, pp[x], o);
                if (lane == 0) {
                    float* orow = out + (size_t)(t0 + t) * ldo + (size_t)h * dv + ew;
#pragma unroll
                    for (int x = 0; x < DC_CW; x++)
                        if (ew + x < dv) orow[x] = pp[x];
                }
            }
        }
        __syncthreads();
    }
    (void)s0row;
    float* dst = OUT ? srow : P + (bh * nc_max + c) * dv * d;
    if (!OUT || last) {
#pragma unroll
        for (int x = 0; x < DC_CW; x++)
#pragma unroll
            for (int i = 0; i < DPL; i++) {
                const int j = lane + 32 * i;
                if (ew + x < dv && j < d) dst[(size_t)(ew + x) * d + j] = S[x][i];
            }
    }
}

// chunked form: C = tokens of a chunk, nc_max = the most chunks a sequence of this step can have (the longest
// sequence's; an upper bound is fine), P (float [B][H][nc_max][dv][d]) and S0 (float [B][H][dv][d]) scratch
// The two passes with a THREAD per column of the state (key sizes up to 128): the thread holds its column's D
// elements in registers, so a token's output is a private sum (no exchange between lanes), k and q of a token are
// read from shared memory as broadcasts of four, and a block's threads write 128 neighbouring outputs. About a third
// of the instructions per token of the warp-per-column form above, which stays for larger key sizes.
#define DK_TILE 16
#define DK_COLS 128
template <typename TIN, bool OUT, int D>
__global__ void __launch_bounds__(DK_COLS) k_decay_chunk_col(const TIN* KB_STEP_DATA in, int n_planes,
        size_t plane_stride, int ld_in, int H, int d, int dv, const float* __restrict__ decay,
        const int* __restrict__ q_start, const int* __restrict__ slot, float* state, float* P, float* S0,
        float* __restrict__ out, int ldo, int C, int nc_max) {
    extern __shared__ __align__(16) float smc[];
    float* qs = smc;                                  // [DK_TILE][D] (zeros past d)
    float* ks = qs + DK_TILE * D;                     // [DK_TILE][D]
    float* vs = ks + DK_TILE * D;                     // [DK_TILE][DK_COLS]
    kb_pdl_launch();
    const int b = blockIdx.x / H, h = blockIdx.x % H, c = blockIdx.z;
    const int e0 = blockIdx.y * DK_COLS, e = e0 + threadIdx.x;
    const bool live = e < dv;
    const int r0 = q_start[b], r1 = q_start[b + 1];
    const int nc = (r1 - r0 + C - 1) / C;
    if (c >= nc) return;
    const bool last = c == nc - 1;
    const float lam = decay[h];
    const size_t bh = (size_t)b * H + h;
    float* srow = state + (((size_t)slot[b] * H + h) * dv + (live ? e : 0)) * d;
    float* s0row = S0 + (bh * dv + (live ? e : 0)) * d;
    float* prow = P + ((bh * nc_max + c) * dv + (live ? e : 0)) * d;
    kb_pdl_wait();
    float S[D];
    if (!OUT) {
        if (c == 0 && live)
            for (int j = 0; j < d; j++) s0row[j] = srow[j];
        if (last) return;
#pragma unroll
        for (int j = 0; j < D; j++) S[j] = 0.0f;
    } else {
#pragma unroll
        for (int j = 0; j < D; j++) S[j] = (live && j < d) ? prow[j] : 0.0f;
    }
    const int ra = r0 + c * C, rz = min(ra + C, r1);
    const size_t oq = (size_t)h * d, ok = (size_t)H * d + (size_t)h * d, ov = (size_t)2 * H * d + (size_t)h * dv;
    // (silu(0) = 0: a zero piece past the row's end or past d stages zeros)
    const bool vec8 = sizeof(TIN) == 2 && n_planes == 1 && d % 8 == 0 && ld_in % 8 == 0 && ((uintptr_t)in & 15) == 0;
    for (int t0 = ra; t0 < rz; t0 += DK_TILE) {
        const int n = min(DK_TILE, rz - t0);
        if (vec8) {
            // bf16 rows whose heads start on 16-byte boundaries: eight elements a load, all of a thread's loads in
            // flight before the first is used
            constexpr int PER = (DK_TILE * D / 8 + DK_COLS - 1) / DK_COLS;
            uint4 rq[PER], rk[PER];
#pragma unroll
            for (int u = 0; u < PER; u++) {
                const int idx = (threadIdx.x + DK_COLS * u) * 8, t = idx / D, j = idx % D;
                rq[u] = rk[u] = make_uint4(0u, 0u, 0u, 0u);
                if (idx < DK_TILE * D && t < n && j < d) {
                    const bf16* src = (const bf16*)in + (size_t)(t0 + t) * ld_in;
                    if (OUT) rq[u] = *(const uint4*)(src + oq + j);
                    rk[u] = *(const uint4*)(src + ok + j);
                }
            }
#pragma unroll
            for (int u = 0; u < PER; u++) {
                const int idx = (threadIdx.x + DK_COLS * u) * 8;
                if (idx >= DK_TILE * D) continue;
                const __nv_bfloat162* q2 = (const __nv_bfloat162*)&rq[u];
                const __nv_bfloat162* k2 = (const __nv_bfloat162*)&rk[u];
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const float2 kf = __bfloat1622float2(k2[w]);
                    ks[idx + 2 * w] = mx_silu_fast(kf.x);
                    ks[idx + 2 * w + 1] = mx_silu_fast(kf.y);
                    if (OUT) {
                        const float2 qf = __bfloat1622float2(q2[w]);
                        qs[idx + 2 * w] = mx_silu_fast(qf.x);
                        qs[idx + 2 * w + 1] = mx_silu_fast(qf.y);
                    }
                }
            }
        } else {
            for (int idx = threadIdx.x; idx < DK_TILE * D; idx += DK_COLS) {
                const int t = idx / D, j = idx % D;
                float qv = 0.0f, kv = 0.0f;
                if (t < n && j < d) {
                    const TIN* src = in + (size_t)(t0 + t) * ld_in;
                    if (OUT) qv = mx_silu_fast(mx_rd<TIN>(src, n_planes, plane_stride, oq + j));
                    kv = mx_silu_fast(mx_rd<TIN>(src, n_planes, plane_stride, ok + j));
                }
                if (OUT) qs[idx] = qv;
                ks[idx] = kv;
            }
        }
        for (int t = 0; t < n; t++)
            vs[t * DK_COLS + threadIdx.x] =
                live ? mx_silu_fast(mx_rd<TIN>(in + (size_t)(t0 + t) * ld_in, n_planes, plane_stride, ov + e)) : 0.0f;
        __syncthreads();
        for (int t = 0; t < n; t++) {
            const float v = vs[t * DK_COLS + threadIdx.x];
            float p0 = 0.0f, p1 = 0.0f;
#pragma unroll
            for (int j = 0; j < D; j += 4) {
                const float4 k4 = *(const float4*)(ks + t * D + j);
                S[j] = fmaf(lam, S[j], __fmul_rn(k4.x, v));
                S[j + 1] = fmaf(lam, S[j + 1], __fmul_rn(k4.y, v));
                S[j + 2] = fmaf(lam, S[j + 2], __fmul_rn(k4.z, v));
                S[j + 3] = fmaf(lam, S[j + 3], __fmul_rn(k4.w, v));
                if (OUT) {
                    const float4 q4 = *(const float4*)(qs + t * D + j);
                    p0 = fmaf(S[j], q4.x, p0);
                    p1 = fmaf(S[j + 1], q4.y, p1);
                    p0 = fmaf(S[j + 2], q4.z, p0);
                    p1 = fmaf(S[j + 3], q4.w, p1);
                }
            }
            if (OUT && live) out[(size_t)(t0 + t) * ldo + (size_t)h * dv + e] = p0 + p1;
        }
        __syncthreads();
    }
    if (live && (!OUT || last)) {
        float* dst = OUT ? srow : prow;
#pragma unroll
        for (int j = 0; j < D; j++)
            if (j < d) dst[j] = S[j];
    }
    (void)s0row;
}

// between the two passes: P[c] (a chunk's own contribution) becomes the state BEFORE chunk c, element by element:
// S = the state the sequence came with; for c = 0, 1, ...: (P[c], S) <- (S, decay^C S + P[c])
__global__ void __launch_bounds__(256) k_decay_prefix(int H, int d, int dv, const float* __restrict__ decay,
        const int* __restrict__ q_start, float* P, const float* S0, int C, int nc_max) {
    kb_pdl_launch();
    const int b = blockIdx.x / H, h = blockIdx.x % H;
    const int nc = (q_start[b + 1] - q_start[b] + C - 1) / C;
    const float lamC = powf(decay[h], (float)C);
    const size_t bh = (size_t)b * H + h, n = (size_t)dv * d;
    kb_pdl_wait();
    for (size_t x = (size_t)blockIdx.y * 256 + threadIdx.x; x < n; x += (size_t)gridDim.y * 256) {
        float S = S0[bh * n + x];
        // (eight chunks' contributions are fetched before the first is used: the loads do not wait for one another)
        for (int c0 = 0; c0 < nc; c0 += 8) {
            float own[8];
#pragma unroll
            for (int u = 0; u < 8; u++)            // (the last chunk's contribution is never needed, nor written)
                own[u] = c0 + u < nc - 1 ? P[(bh * nc_max + c0 + u) * n + x] : 0.0f;
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (c0 + u < nc) {
                    P[(bh * nc_max + c0 + u) * n + x] = S;
                    S = fmaf(lamC, S, own[u]);
                }
        }
    }
}

extern "C" int kb_decay_chunked(const void* in, int in_dtype, int n_planes, long long plane_stride, int ld_in, int B,
                                int H, int d, int dv, const float* decay, const int* q_start, const int* slot,
                                float* state, float* P, float* S0, float* out, int ldo, int C, int nc_max,
                                cudaStream_t st) {
    if (B <= 0 || H <= 0 || nc_max <= 0) return 0;
    if (d > 32 * DS_MAX_DPL || d <= 0 || dv <= 0 || C <= 0 || nc_max > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid(B * H, (dv + DC_COLS - 1) / DC_COLS, nc_max);
    dim3 gk(B * H, (dv + DK_COLS - 1) / DK_COLS, nc_max);
    dim3 gs(B * H, (unsigned)((dv * d + 255) / 256 < 64 ? (dv * d + 255) / 256 : 64));
#define KB_DC2(TIN, DPL)                                                                                            \
    do {                                                                                                            \
        const size_t sm = (size_t)(2 * DC_TILE * 32 * DPL + DC_TILE * DC_COLS) * sizeof(float);                     \
        kb_launch(k_decay_chunk<TIN, false, DPL>, grid, 256, sm, st, (const TIN*)in, n_planes,                     \
                  (size_t)plane_stride, ld_in, H, d, dv, decay, q_start, slot, state, P, S0, out, ldo, C, nc_max);  \
        cudaError_t e = cudaGetLastError();                                                                         \
        if (e != cudaSuccess) return (int)e;                                                                        \
        kb_launch(k_decay_prefix, gs, 256, 0, st, H, d, dv, decay, q_start, P, (const float*)S0, C, nc_max);        \
        e = cudaGetLastError();                                                                                     \
        if (e != cudaSuccess) return (int)e;                                                                        \
        kb_launch(k_decay_chunk<TIN, true, DPL>, grid, 256, sm, st, (const TIN*)in, n_planes,                      \
                  (size_t)plane_stride, ld_in, H, d, dv, decay, q_start, slot, state, P, S0, out, ldo, C, nc_max);  \
    } while (0)
#define KB_DK2(TIN, D)                                                                                              \
    do {                                                                                                            \
        const size_t sm = (size_t)(2 * DK_TILE * D + DK_TILE * DK_COLS) * sizeof(float);                            \
        kb_launch(k_decay_chunk_col<TIN, false, D>, gk, DK_COLS, sm, st, (const TIN*)in, n_planes,                  \
                  (size_t)plane_stride, ld_in, H, d, dv, decay, q_start, slot, state, P, S0, out, ldo, C, nc_max);  \
        cudaError_t e = cudaGetLastError();                                                                         \
        if (e != cudaSuccess) return (int)e;                                                                        \
        kb_launch(k_decay_prefix, gs, 256, 0, st, H, d, dv, decay, q_start, P, (const float*)S0, C, nc_max);        \
        e = cudaGetLastError();                                                                                     \
        if (e != cudaSuccess) return (int)e;                                                                        \
        kb_launch(k_decay_chunk_col<TIN, true, D>, gk, DK_COLS, sm, st, (const TIN*)in, n_planes,                   \
                  (size_t)plane_stride, ld_in, H, d, dv, decay, q_start, slot, state, P, S0, out, ldo, C, nc_max);  \
    } while (0)
#define KB_DC(TIN)                          \
    do {                                    \
        if (d <= 32) KB_DK2(TIN, 32);       \
        else if (d <= 64) KB_DK2(TIN, 64);  \
        else if (d <= 128) KB_DK2(TIN, 128);\
        else KB_DC2(TIN, 8);                \
    } while (0)
    if (in_dtype == KB_F32) KB_DC(float);
    else KB_DC(bf16);
#undef KB_DK2
#undef KB_DC2
#undef KB_DC
    KB_LAUNCH_RET();
}

extern "C" int kb_decay_scan(const void* in, int in_dtype, int n_planes, long long plane_stride, int ld_in, int B,
                             int H, int d, int dv, const float* decay, const int* q_start, const int* slot, float* state,
                             float* out, int ldo, cudaStream_t st) {
    if (B <= 0 || H <= 0) return 0;
    if (d > 32 * DS_MAX_DPL || d <= 0 || dv <= 0) return (int)cudaErrorInvalidValue;
    dim3 grid(B * H, (dv + DS_COLS - 1) / DS_COLS);
    const size_t sm = (size_t)(2 * DS_CHUNK * d + DS_CHUNK * DS_COLS) * sizeof(float);
    if (in_dtype == KB_F32)
        kb_launch(k_decay_scan<float>, grid, 32 * DS_COLS, sm, st, (const float*)in, n_planes, (size_t)plane_stride,
                  ld_in, H, d, dv, decay, q_start, slot, state, out, ldo);
    else
        kb_launch(k_decay_scan<bf16>, grid, 32 * DS_COLS, sm, st, (const bf16*)in, n_planes, (size_t)plane_stride, ld_in,
                  H, d, dv, decay, q_start, slot, state, out, ldo);
    KB_LAUNCH_RET();
}
