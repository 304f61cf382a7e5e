// Layer norm with the residual add fused in front of it, and the plain residual add.
//
// k_add_layernorm: row r of the output is row t = rows ? rows[r] : r of the residual. v = x[t] + sum_s delta[s][t]
// (s in order), written back to x when write_back; mean = sum(v) / E; var = sum((v - mean)^2) / E (the mean of the
// squared deviations, taken in a second pass over the row, which the block keeps in shared memory);
// y = (v - mean) / sqrt(var + eps) * w + b. Everything is 32-bit; a row's sums are taken by a fixed number of
// threads in a fixed order, so a row gives the same bits whatever else the step holds.
//
// k_residual_add: x += sum_s delta[s] (s in order) + extra, element by element: what a model that feeds its embedding
// output into the residual stream again needs between two layers.
#include "common.cuh"

#define LN_THREADS 512
#define LN_MAX_E 51200

__device__ __forceinline__ float ln_block_sum(float v, float* red) {
    v = kb_warp_sum(v);
    __syncthreads();                                 // red may still be read from the sum before
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = red[0];
#pragma unroll
    for (int k = 1; k < LN_THREADS / 32; k++) tot += red[k];
    return tot;
}

template <typename TY, typename TW>
__global__ void __launch_bounds__(LN_THREADS) k_add_layernorm(float* KB_STEP_DATA x, const float* KB_STEP_DATA delta,
        int n_delta, size_t delta_stride, const TW* __restrict__ w, const TW* __restrict__ bias, float eps,
        TY* __restrict__ y, const int* __restrict__ rows, int T, int E, int write_back, int vec, int* status) {
    extern __shared__ float sv[];
    __shared__ float red[LN_THREADS / 32];
    kb_pdl_launch();
    const int r = blockIdx.x;
    int t = rows ? rows[r] : r;
    if (t < 0 || t >= T) {
        if (threadIdx.x == 0) atomicOr(status, KB_ST_BAD_ROW);
        t = 0;
    }
    float* xr = x + (size_t)t * E;
    const float* dr = delta + (size_t)t * E;
    kb_pdl_wait();
    float s = 0.0f;
    if (vec) {
        for (int i = threadIdx.x * 4; i < E; i += LN_THREADS * 4) {
            float4 v = *(const float4*)(xr + i);
            for (int p = 0; p < n_delta; p++) {
                const float4 d = *(const float4*)(dr + (size_t)p * delta_stride + i);
                v.x += d.x;
                v.y += d.y;
                v.z += d.z;
                v.w += d.w;
            }
            if (write_back) *(float4*)(xr + i) = v;
            *(float4*)(sv + i) = v;
            s += (v.x + v.y) + (v.z + v.w);
        }
    } else {
        for (int i = threadIdx.x; i < E; i += LN_THREADS) {
            float v = xr[i];
            for (int p = 0; p < n_delta; p++) v += dr[(size_t)p * delta_stride + i];
            if (write_back) xr[i] = v;
            sv[i] = v;
            s += v;
        }
    }
    const float mean = ln_block_sum(s, red) / (float)E;
    float q = 0.0f;
    if (vec) {
        for (int i = threadIdx.x * 4; i < E; i += LN_THREADS * 4) {
            const float4 v = *(const float4*)(sv + i);
            const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
            q += (a * a + b * b) + (c * c + d * d);
        }
    } else {
        for (int i = threadIdx.x; i < E; i += LN_THREADS) {
            const float a = sv[i] - mean;
            q = fmaf(a, a, q);
        }
    }
    const float var = ln_block_sum(q, red) / (float)E;
    const float inv = 1.0f / sqrtf(var + eps);
    TY* yr = y + (size_t)r * E;
    for (int i = threadIdx.x; i < E; i += LN_THREADS)
        yr[i] = kb_from_f<TY>(__fadd_rn(__fmul_rn(__fmul_rn(sv[i] - mean, inv), kb_to_f<TW>(w[i])),
                                        kb_to_f<TW>(bias[i])));
}

// The same operation with one warp per row and the row in registers, for prompt-sized steps of the bfloat16 path: no
// shared memory, no block barrier. Its sums are taken in another order than k_add_layernorm's, so the true 32-bit path,
// whose results must not depend on how many rows a step has, never uses it. NC float4 per lane: widths up to 128 * NC
// (up to 2048: at 4096 the row no longer fits the registers of enough resident warps, and the block per row is faster).
#define LN_WARP_MIN_T 64
template <typename TW, int NC>
__global__ void __launch_bounds__(256) k_add_layernorm_warp(float* KB_STEP_DATA x, const float* KB_STEP_DATA delta,
        int n_delta, size_t delta_stride, const TW* __restrict__ w, const TW* __restrict__ bias, float eps,
        bf16* __restrict__ y, int T, int E, int write_back) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= T) return;
    float* xr = x + (size_t)t * E;
    const float* dr = delta + (size_t)t * E;
    float4 v[NC];
    float s = 0.0f;
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const int i = (c * 32 + lane) * 4;
        v[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < E) {
            v[c] = *(const float4*)(xr + i);
            for (int p = 0; p < n_delta; p++) {
                const float4 d = *(const float4*)(dr + (size_t)p * delta_stride + i);
                v[c].x += d.x;
                v[c].y += d.y;
                v[c].z += d.z;
                v[c].w += d.w;
            }
            if (write_back) *(float4*)(xr + i) = v[c];
            s += (v[c].x + v[c].y) + (v[c].z + v[c].w);
        }
    }
    const float mean = kb_warp_sum(s) / (float)E;
    float q = 0.0f;
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const int i = (c * 32 + lane) * 4;
        if (i < E) {
            const float a = v[c].x - mean, b = v[c].y - mean, cc = v[c].z - mean, d = v[c].w - mean;
            q += (a * a + b * b) + (cc * cc + d * d);
        }
    }
    const float inv = 1.0f / sqrtf(kb_warp_sum(q) / (float)E + eps);
    bf16* yr = y + (size_t)t * E;
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const int i = (c * 32 + lane) * 4;
        if (i < E) {
            const float o0 = __fadd_rn(__fmul_rn(__fmul_rn(v[c].x - mean, inv), kb_to_f<TW>(w[i])), kb_to_f<TW>(bias[i]));
            const float o1 = __fadd_rn(__fmul_rn(__fmul_rn(v[c].y - mean, inv), kb_to_f<TW>(w[i + 1])), kb_to_f<TW>(bias[i + 1]));
            const float o2 = __fadd_rn(__fmul_rn(__fmul_rn(v[c].z - mean, inv), kb_to_f<TW>(w[i + 2])), kb_to_f<TW>(bias[i + 2]));
            const float o3 = __fadd_rn(__fmul_rn(__fmul_rn(v[c].w - mean, inv), kb_to_f<TW>(w[i + 3])), kb_to_f<TW>(bias[i + 3]));
            __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
            *(uint2*)(yr + i) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
        }
    }
}

extern "C" int kb_add_layernorm(float* x, const float* delta, int n_delta, long long delta_stride, const void* w,
                                const void* bias, int wdtype, float eps, void* y, int ydtype, const int* rows,
                                int n_out, int T, int E, int write_back, int* status, cudaStream_t st) {
    if (n_out <= 0) return 0;
    if (E > LN_MAX_E) return (int)cudaErrorInvalidValue;
    const size_t sm = (size_t)E * sizeof(float);
    const int vec = (E % 4 == 0) && (((uintptr_t)x) % 16 == 0) && (((uintptr_t)delta) % 16 == 0) &&
                    (delta_stride % 4 == 0);
    cudaError_t e = cudaSuccess;
    if (ydtype == KB_BF16 && vec && rows == nullptr && n_out == T && T >= LN_WARP_MIN_T && E <= 128 * 16 &&
        (write_back || n_delta == 0) && (((uintptr_t)y) % 8) == 0) {
#define KB_LNW(NC)                                                                                                 \
    do {                                                                                                           \
        if (wdtype == KB_F32)                                                                                      \
            e = kb_launch(k_add_layernorm_warp<float, NC>, (T + 7) / 8, 256, 0, st, x, delta, n_delta,             \
                          (size_t)delta_stride, (const float*)w, (const float*)bias, eps, (bf16*)y, T, E,          \
                          write_back);                                                                             \
        else                                                                                                       \
            e = kb_launch(k_add_layernorm_warp<bf16, NC>, (T + 7) / 8, 256, 0, st, x, delta, n_delta,              \
                          (size_t)delta_stride, (const bf16*)w, (const bf16*)bias, eps, (bf16*)y, T, E,            \
                          write_back);                                                                             \
        return (int)e;                                                                                             \
    } while (0)
        if (E <= 128 * 4) KB_LNW(4);
        if (E <= 128 * 8) KB_LNW(8);
        KB_LNW(16);
#undef KB_LNW
    }
#define KB_LN(TY, TW)                                                                                              \
    do {                                                                                                           \
        if (sm > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(k_add_layernorm<TY, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);   \
        e = kb_launch(k_add_layernorm<TY, TW>, n_out, LN_THREADS, sm, st, x, delta, n_delta, (size_t)delta_stride, \
                      (const TW*)w, (const TW*)bias, eps, (TY*)y, rows, T, E, write_back, vec, status);            \
    } while (0)
    if (ydtype == KB_F32 && wdtype == KB_F32) KB_LN(float, float);
    else if (ydtype == KB_F32) KB_LN(float, bf16);
    else if (wdtype == KB_F32) KB_LN(bf16, float);
    else KB_LN(bf16, bf16);
#undef KB_LN
    return (int)e;
}

__global__ void __launch_bounds__(256) k_residual_add(float* KB_STEP_DATA x, const float* KB_STEP_DATA delta,
        int n_delta, size_t delta_stride, const float* KB_STEP_DATA extra, long long n) {
    kb_pdl_launch();
    kb_pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = x[i];
        for (int p = 0; p < n_delta; p++) v += delta[(size_t)p * delta_stride + i];
        if (extra) v += extra[i];
        x[i] = v;
    }
}

extern "C" int kb_residual_add(float* x, const float* delta, int n_delta, long long delta_stride, const float* extra,
                               long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const long long want = (n + 255) / 256;
    const int blocks = (int)(want < 4736 ? want : 4736);
    kb_launch(k_residual_add, blocks, 256, 0, st, x, delta, n_delta, (size_t)delta_stride, extra, n);
    KB_LAUNCH_RET();
}
