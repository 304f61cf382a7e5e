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

// ---- eight elements at a time -------------------------------------------------------------------------------------
__device__ __forceinline__ void qn_load8(const float* p, float* o) {
    const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void qn_load8(const bf16* p, float* o) {
    const uint4 r = *(const uint4*)p;
    const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        o[2 * j] = __uint_as_float(u[j] << 16);
        o[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
    }
}
__device__ __forceinline__ void qn_store8(float* p, const float* v) {
    *(float4*)p = make_float4(v[0], v[1], v[2], v[3]);
    *(float4*)(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void qn_store8(bf16* p, const float* v) {
    uint32_t h[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        h[j] = *(uint32_t*)&t;
    }
    *(uint4*)p = make_uint4(h[0], h[1], h[2], h[3]);
}

// The same operation for rows whose pieces are aligned (head size and half the rotated dimensions multiples of 8, rows
// and pages 16-byte aligned): every load and store moves eight elements, the gains are applied where the values are
// rotated (no pass of its own), and a thread rotates eight pairs at a time. Each value is computed by the expressions
// of k_norm_rope_store, so both give the same bits.
template <typename TIN, typename T, typename TW>
__global__ void __launch_bounds__(QN_THREADS) k_norm_rope_store8(const TIN* KB_STEP_DATA in, int n_planes,
        size_t plane_stride, int ld_in, T* qout, int ldq, const TW* __restrict__ wq,
        const TW* __restrict__ wk, float eps, int nq_true, int nk_true, const float* __restrict__ inv_freq, int rot,
        const int* __restrict__ pos, const int* __restrict__ seq, const int* __restrict__ slot, int nh, int nkv,
        int nkv_store, int hd, KbCacheView cv, int* status) {
    extern __shared__ __align__(16) float sm8[];
    __shared__ float2 red[QN_THREADS / 32];
    kb_pdl_launch();
    const int t = blockIdx.x;
    const int p = pos[t];
    if (p < 0) return;
    const int half = rot / 2;
    const int n_q = nh * hd, n_k = nkv * hd, n_all = n_q + 2 * n_k;
    float* row = sm8;
    float2* cs = (float2*)(sm8 + n_all);
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
    for (int i = threadIdx.x * 8; i < n_all; i += QN_THREADS * 8) {
        float v[8];
        qn_load8(src + i, v);
        for (int s = 1; s < n_planes; s++) {
            float d[8];
            qn_load8(src + (size_t)s * plane_stride + i, d);
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] += d[j];
        }
        qn_store8(row + i, v);
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; j++) ss = fmaf(v[j], v[j], ss);
        if (i < n_q) sq += ss;
        else if (i < n_q + n_k) sk += ss;
    }
    const float2 tot = qn_block_sum2(sq, sk, red);
    const bool normed = wq != nullptr;
    const float fq = normed ? 1.0f / sqrtf(tot.x / (float)nq_true + eps) : 1.0f;
    const float fk = normed ? 1.0f / sqrtf(tot.y / (float)nk_true + eps) : 1.0f;
    // query and key heads: per head, half / 8 items that rotate eight pairs, then (hd - rot) / 8 items that pass on
    const int n_rot = half / 8, per_head = n_rot + (hd - rot) / 8;
    const int n_qk = nh + (page >= 0 ? nkv_store : 0);
    for (int e = threadIdx.x; e < n_qk * per_head; e += QN_THREADS) {
        const int h = e / per_head, it = e % per_head;
        const bool is_q = h < nh;
        const int hk = h - nh;
        T* dst = is_q ? qout + (size_t)t * ldq + (size_t)h * hd
                      : (T*)cv.pool + kb_kv_offset(cv, page, 0, hk, p % KB_PAGE);
        const int base = is_q ? h * hd : n_q + hk * hd;                 // the head's place in the row
        const TW* g = normed ? (is_q ? wq + h * hd : wk + hk * hd) : nullptr;
        const float f = is_q ? fq : fk;
        if (it < n_rot) {
            const int i = it * 8;
            float a[8], b[8], ga[8], gb[8], lo[8], hi[8];
            qn_load8(row + base + i, a);
            qn_load8(row + base + i + half, b);
            if (normed) {
                qn_load8(g + i, ga);
                qn_load8(g + i + half, gb);
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float x = normed ? __fmul_rn(__fmul_rn(a[j], f), ga[j]) : a[j];
                const float y = normed ? __fmul_rn(__fmul_rn(b[j], f), gb[j]) : b[j];
                const float2 c = cs[i + j];
                lo[j] = __fsub_rn(__fmul_rn(x, c.x), __fmul_rn(y, c.y));
                hi[j] = __fadd_rn(__fmul_rn(y, c.x), __fmul_rn(x, c.y));
            }
            qn_store8(dst + i, lo);
            qn_store8(dst + i + half, hi);
        } else {
            const int i = rot + (it - n_rot) * 8;
            float a[8], ga[8];
            qn_load8(row + base + i, a);
            if (normed) {
                qn_load8(g + i, ga);
#pragma unroll
                for (int j = 0; j < 8; j++) a[j] = __fmul_rn(__fmul_rn(a[j], f), ga[j]);
            }
            qn_store8(dst + i, a);
        }
    }
    if (page >= 0) {
        const int per_v = hd / 8;
        for (int e = threadIdx.x; e < nkv_store * per_v; e += QN_THREADS) {
            const int hk = e / per_v, i = (e % per_v) * 8;
            float a[8];
            qn_load8(row + n_q + n_k + hk * hd + i, a);
            qn_store8((T*)cv.pool + kb_kv_offset(cv, page, 1, hk, p % KB_PAGE) + i, a);
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
    const int in_el = in_dtype == KB_F32 ? 4 : 2, out_el = dtype == KB_F32 ? 4 : 2, w_el = wdtype == KB_F32 ? 4 : 2;
    const bool by8 = hd % 8 == 0 && rot % 16 == 0 && ld_in % 8 == 0 && ldq % 8 == 0 && plane_stride % 8 == 0 &&
                     ((uintptr_t)in % (8 * in_el)) == 0 && ((uintptr_t)qout % (8 * out_el)) == 0 &&
                     ((uintptr_t)pool % (8 * out_el)) == 0 && ((uintptr_t)wq % (8 * w_el)) == 0 &&
                     ((uintptr_t)wk % (8 * w_el)) == 0;
#define KB_QN8(TIN, T_, TW)                                                                                        \
    do {                                                                                                           \
        if (smem > 48 * 1024)                                                                                      \
            cudaFuncSetAttribute(k_norm_rope_store8<TIN, T_, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                 (int)smem);                                                                       \
        e = kb_launch(k_norm_rope_store8<TIN, T_, TW>, T, QN_THREADS, smem, st, (const TIN*)in, n_planes,          \
                      (size_t)plane_stride, ld_in, (T_*)qout, ldq, (const TW*)wq, (const TW*)wk, eps, nq_true,     \
                      nk_true, inv_freq, rot, pos, seq, slot, nh, nkv, nkv_store, hd, cv, status);                 \
        return (int)e;                                                                                             \
    } while (0)
    if (by8) {
        if (in_dtype == KB_F32 && dtype == KB_F32 && wdtype == KB_F32) KB_QN8(float, float, float);
        else if (in_dtype == KB_F32 && dtype == KB_F32) KB_QN8(float, float, bf16);
        else if (in_dtype == KB_F32 && dtype == KB_BF16 && wdtype == KB_BF16) KB_QN8(float, bf16, bf16);
        else if (in_dtype == KB_F32 && dtype == KB_BF16) KB_QN8(float, bf16, float);
        else if (in_dtype == KB_BF16 && dtype == KB_BF16 && wdtype == KB_BF16) KB_QN8(bf16, bf16, bf16);
        else if (in_dtype == KB_BF16 && dtype == KB_BF16) KB_QN8(bf16, bf16, float);
    }
#undef KB_QN8
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
