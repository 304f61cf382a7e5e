// Query/key norm over the whole projection, rotation and the key/value store, one block per row.
//
// The row is [q heads | k heads | v heads], every head hd wide, as rows in the run dtype or as 32-bit planes that are
// summed in order. With gains (wq, wk) the query part and the key part are each divided by their root mean square
// over ALL their heads at once - sqrt(sum(v^2) / n_true + eps), n_true being the number of elements the model's
// projection has (heads that were widened with zero rows to the cache's head size count with their true size) - and
// multiplied by the gains, before the rotation. Then, as in k_rope_store: pairs (i, i + rot/2) of every query and key
// head are rotated by pos * inv_freq[i], queries go to qout, keys and values to the row's place in its cache page.
// All of it is 32-bit; each value is rounded to the run dtype once, when it is written.
#include "common.cuh"

#define QN_THREADS 256

__device__ __forceinline__ float2 qn_block_sum2(float a, float b, float2* red) {
    a = kb_warp_sum(a);
    b = kb_warp_sum(b);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = make_float2(a, b);
    __syncthreads();
    float2 tot = red[0];
#pragma unroll
    for (int k = 1; k < QN_THREADS / 32; k++) {
        tot.x += red[k].x;
        tot.y += red[k].y;
    }
    return tot;
}

template <typename TIN, typename T, typename TW>
__global__ void __launch_bounds__(QN_THREADS) k_norm_rope_store(const TIN* KB_STEP_DATA in, int n_planes,
        size_t plane_stride, int ld_in, T* qout, int ldq, const TW* __restrict__ wq,
        const TW* __restrict__ wk, float eps, int nq_true, int nk_true, const float* __restrict__ inv_freq, int rot,
        const int* __restrict__ pos, const int* __restrict__ seq, const int* __restrict__ slot, int nh, int nkv,
        int nkv_store, int hd, KbCacheView cv, int* status) {
    extern __shared__ float sm[];
    __shared__ float2 red[QN_THREADS / 32];
    kb_pdl_launch();
    const int t = blockIdx.x;
    const int p = pos[t];
    if (p < 0) return;                               // a padding row of a recorded step
    const int half = rot / 2;
    const int n_q = nh * hd, n_k = nkv * hd, n_all = n_q + 2 * n_k;
    float* row = sm;                                 // [n_all]
    float2* cs = (float2*)(sm + ((n_all + 1) & ~1)); // [half]: cosine and sine of the row's angles
    int page = -1;
    if (nkv_store > 0) {
        const int s = slot[seq[t]];
        page = cv.table[(size_t)s * cv.table_stride + p / KB_PAGE];
        if (page < 0 || page >= cv.n_pages) page = -1;
    }
    for (int i = threadIdx.x; i < half; i += QN_THREADS) {
        const float ang = __fmul_rn((float)p, inv_freq[i]);
        cs[i] = make_float2(cosf(ang), sinf(ang));
    }
    kb_pdl_wait();
    if (nkv_store > 0 && page < 0 && threadIdx.x == 0) atomicOr(status, KB_ST_BAD_PAGE);
    const TIN* src = in + (size_t)t * ld_in;
    float sq = 0.0f, sk = 0.0f;
    for (int i = threadIdx.x; i < n_all; i += QN_THREADS) {
        float v = kb_to_f<TIN>(src[i]);
        for (int s = 1; s < n_planes; s++) v += kb_to_f<TIN>(src[(size_t)s * plane_stride + i]);
        row[i] = v;
        if (i < n_q) sq = fmaf(v, v, sq);
        else if (i < n_q + n_k) sk = fmaf(v, v, sk);
    }
    const float2 tot = qn_block_sum2(sq, sk, red);   // (its barrier also makes the row and the angles visible)
    if (wq != nullptr) {
        const float fq = 1.0f / sqrtf(tot.x / (float)nq_true + eps), fk = 1.0f / sqrtf(tot.y / (float)nk_true + eps);
        for (int i = threadIdx.x; i < n_q + n_k; i += QN_THREADS)
            row[i] = i < n_q ? __fmul_rn(__fmul_rn(row[i], fq), kb_to_f<TW>(wq[i]))
                             : __fmul_rn(__fmul_rn(row[i], fk), kb_to_f<TW>(wk[i - n_q]));
        __syncthreads();
    }
    // queries and keys: element (head h, index i < hd); a thread takes the pair (i, i + half) when i < half, the
    // element alone when i >= rot
    const int n_heads_out = nh + (page >= 0 ? 2 * nkv_store : 0);
    for (int e = threadIdx.x; e < n_heads_out * hd; e += QN_THREADS) {
        const int h = e / hd, i = e % hd;
        T* dst;
        const float* srow;
        bool rotate = true;
        if (h < nh) {
            dst = qout + (size_t)t * ldq + (size_t)h * hd;
            srow = row + (size_t)h * hd;
        } else if (h < nh + nkv_store) {
            const int hk = h - nh;
            dst = (T*)cv.pool + kb_kv_offset(cv, page, 0, hk, p % KB_PAGE);
            srow = row + n_q + (size_t)hk * hd;
        } else {
            const int hk = h - nh - nkv_store;
            dst = (T*)cv.pool + kb_kv_offset(cv, page, 1, hk, p % KB_PAGE);
            srow = row + n_q + n_k + (size_t)hk * hd;
            rotate = false;
        }
        if (!rotate || i >= rot) {
            dst[i] = kb_from_f<T>(srow[i]);
        } else if (i < half) {
            const float a = srow[i], b = srow[i + half];
            const float2 c = cs[i];
            dst[i] = kb_from_f<T>(__fsub_rn(__fmul_rn(a, c.x), __fmul_rn(b, c.y)));
            dst[i + half] = kb_from_f<T>(__fadd_rn(__fmul_rn(b, c.x), __fmul_rn(a, c.y)));
        }
    }
}

extern "C" int kb_norm_rope_store(const void* in, int in_dtype, int n_planes, long long plane_stride, int ld_in,
                                  void* qout, int dtype, int ldq, const void* wq, const void* wk, int wdtype,
                                  float eps, int nq_true, int nk_true, const float* inv_freq, int rot, const int* pos,
                                  const int* seq, const int* slot, int T, int nh, int nkv, int nkv_store, int hd,
                                  void* pool, const int* table, int table_stride, int n_pages, int* status,
                                  cudaStream_t st) {
    if (T <= 0) return 0;
    KbCacheView cv{pool, table, table_stride, n_pages, nkv, hd};
    const int n_all = (nh + 2 * nkv) * hd;
    const size_t smem = (size_t)((n_all + 1) & ~1) * sizeof(float) + (size_t)(rot / 2) * sizeof(float2);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaSuccess;
#define KB_QN(TIN, T_, TW)                                                                                         \
    do {                                                                                                           \
        if (smem > 48 * 1024)                                                                                      \
            cudaFuncSetAttribute(k_norm_rope_store<TIN, T_, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                 (int)smem);                                                                       \
        e = kb_launch(k_norm_rope_store<TIN, T_, TW>, T, QN_THREADS, smem, st, (const TIN*)in, n_planes,           \
                      (size_t)plane_stride, ld_in, (T_*)qout, ldq, (const TW*)wq, (const TW*)wk, eps, nq_true,     \
                      nk_true, inv_freq, rot, pos, seq, slot, nh, nkv, nkv_store, hd, cv, status);                 \
    } while (0)
    if (in_dtype == KB_F32 && dtype == KB_F32 && wdtype == KB_F32) KB_QN(float, float, float);
    else if (in_dtype == KB_F32 && dtype == KB_F32) KB_QN(float, float, bf16);
    else if (in_dtype == KB_F32 && dtype == KB_BF16 && wdtype == KB_BF16) KB_QN(float, bf16, bf16);
    else if (in_dtype == KB_F32 && dtype == KB_BF16) KB_QN(float, bf16, float);
    else if (in_dtype == KB_BF16 && dtype == KB_BF16 && wdtype == KB_BF16) KB_QN(bf16, bf16, bf16);
    else if (in_dtype == KB_BF16 && dtype == KB_BF16) KB_QN(bf16, bf16, float);
    else return (int)cudaErrorInvalidValue;
#undef KB_QN
    return (int)e;
}
