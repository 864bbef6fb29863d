// Steps around the sublayers of a decoder whose norm sits on a sublayer's OUTPUT, and an embedding with a second, hashed row.
//
//  embed_hashed       x[t] = E[id_t] + B[row_t];  row_t = (id_(t-1) a + id_t b) mod n, and row n for a request's first token.  The token
//                     before a step's first one is a word of the request's state slot; the block of a segment's first token reads
//                     it and then writes the segment's last token there (nobody else touches the word).
//  residual_norm_step x[t] += m * (y[t] / sqrt(mean(y[t]^2) + eps)) * w;  y[t] <- 0;  xc[t] <- x[t] in the compute dtype (if asked).
//                     Without w nothing is added: y is zeroed and xc written, which is how a pass begins.
//                     One block a row; what a sublayer ADDED into the zeroed y is normed, scaled and summed into the float32
//                     residual row, y is zero again for the next sublayer, and the next sublayer's input is written.
//  glu_clamped        out = g' sigmoid(alpha g') (u' + 1),  g' = min(g, L),  u' = clamp(u, -L, L);  gu [T, 2I] -> out [T, I].
//
// All arithmetic is float32; accurate expf, division and sqrtf.
#include "common.cuh"

namespace vk {

template <typename T>
__global__ void __launch_bounds__(256) embed_hashed_kernel(const T* __restrict__ table, const T* __restrict__ second, const int32_t* __restrict__ ids,
                                                           const int32_t* __restrict__ positions, const int32_t* __restrict__ token_seg,
                                                           const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots,
                                                           int32_t* __restrict__ last_token, float* __restrict__ x, T* __restrict__ xc, int hidden,
                                                           int vocab, int buckets, int mul_prev, int mul_cur) {
    __shared__ int row_s;
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;          // the host has checked the range; never read outside the table
    if (threadIdx.x == 0) {
        const int seg = token_seg[t];
        const int first = seg_starts[seg], slot = seg_slots[seg];
        int prev = 0;
        if (t > first) prev = ids[t - 1];
        else if (slot >= 0) {
            prev = last_token[slot];
            int last = ids[seg_starts[seg + 1] - 1];
            last_token[slot] = last;
        }
        if (prev < 0 || prev >= vocab) prev = 0;
        row_s = positions[t] == 0 ? buckets : (int)(((long long)prev * mul_prev + (long long)id * mul_cur) % buckets);
    }
    __syncthreads();
    const T* a = table + (size_t)id * hidden;
    float* out = x + (size_t)t * hidden;
    if (second) {
        const T* b = second + (size_t)row_s * hidden;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = to_f32<T>(a[i]) + to_f32<T>(b[i]);
            out[i] = v;
            if (xc) xc[(size_t)t * hidden + i] = from_f32<T>(v);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = to_f32<T>(a[i]);
            out[i] = v;
            if (xc) xc[(size_t)t * hidden + i] = from_f32<T>(v);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) residual_norm_step_kernel(float* __restrict__ x, float* __restrict__ y, const float* __restrict__ w,
                                                                 T* __restrict__ xc, int n, float eps, float mult) {
    __shared__ float scratch[32];
    dependency_wait();
    let_dependents_start();
    const size_t base = (size_t)blockIdx.x * n;
    if (!w) {                                   // the form that starts a pass: nothing is added
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            if (y) y[base + i] = 0.0f;
            if (xc) xc[base + i] = from_f32<T>(x[base + i]);
        }
        return;
    }
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = y[base + i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = x[base + i] + mult * ((y[base + i] * inv) * w[i]);
        x[base + i] = v;
        y[base + i] = 0.0f;
        if (xc) xc[base + i] = from_f32<T>(v);
    }
}

// The step between two sublayers of a layer with a norm before AND behind each sublayer (layer norms with weight and bias):
//   x += LN(y; w_post, b_post),  y = 0,  xn = LN(x; w_next, b_next) in the compute dtype
// (w_post null: nothing is added, y is only zeroed; w_next null: no normed output).  A block a row; the row's values stay in
// registers (up to SW_KEEP a thread) between the sums, which meet in an order that depends on the width alone.
constexpr int SW_THREADS = 128;
constexpr int SW_KEEP = 16;

template <typename T> __device__ __forceinline__ void sw_store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void sw_store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void sw_store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}

// Rows whose width is a multiple of four, of up to 4 * SW_THREADS * SW_VEC values, with every pointer on 16 bytes: all of a thread's
// 16-byte pieces of y and x are asked for before any is used, and stay in registers.  The sums meet in the order of the scalar form's
// block_sum; a thread's own partial sums run over other elements, so the two forms agree to rounding, and which form a row takes
// depends on the width and the buffers alone, never on the batch.
constexpr int SW_VEC = 4;
template <typename T>
__device__ __forceinline__ void sandwich_row_vec(float* __restrict__ x, float* __restrict__ y, const float* __restrict__ wp, const float* __restrict__ bp,
                                                 const float* __restrict__ wn, const float* __restrict__ bn, T* __restrict__ xn, int n, float eps,
                                                 float* scratch) {
    const int tid = threadIdx.x;
    float4 v[SW_VEC], u[SW_VEC];
#pragma unroll
    for (int j = 0; j < SW_VEC; j++) {
        const int i = (tid + j * SW_THREADS) * 4;
        u[j] = i < n ? *reinterpret_cast<const float4*>(x + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        v[j] = (wp && i < n) ? *reinterpret_cast<const float4*>(y + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    if (wp) {
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < SW_VEC; j++) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        const float mean = block_sum(sum, scratch) / (float)n;
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < SW_VEC; j++)
            if ((tid + j * SW_THREADS) * 4 < n) {
                const float d0 = v[j].x - mean, d1 = v[j].y - mean, d2 = v[j].z - mean, d3 = v[j].w - mean;
                ss = fmaf(d0, d0, ss); ss = fmaf(d1, d1, ss); ss = fmaf(d2, d2, ss); ss = fmaf(d3, d3, ss);
            }
        const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
#pragma unroll
        for (int j = 0; j < SW_VEC; j++) {
            const int i = (tid + j * SW_THREADS) * 4;
            if (i < n) {
                const float4 w4 = *reinterpret_cast<const float4*>(wp + i), b4 = *reinterpret_cast<const float4*>(bp + i);
                u[j].x += fmaf((v[j].x - mean) * inv, w4.x, b4.x);
                u[j].y += fmaf((v[j].y - mean) * inv, w4.y, b4.y);
                u[j].z += fmaf((v[j].z - mean) * inv, w4.z, b4.z);
                u[j].w += fmaf((v[j].w - mean) * inv, w4.w, b4.w);
                *reinterpret_cast<float4*>(x + i) = u[j];
            }
        }
    }
    if (y) {
#pragma unroll
        for (int j = 0; j < SW_VEC; j++) {
            const int i = (tid + j * SW_THREADS) * 4;
            if (i < n) *reinterpret_cast<float4*>(y + i) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
    if (!wn) return;
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < SW_VEC; j++) sum += (u[j].x + u[j].y) + (u[j].z + u[j].w);
    const float mean = block_sum(sum, scratch) / (float)n;
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < SW_VEC; j++)
        if ((tid + j * SW_THREADS) * 4 < n) {
            const float d0 = u[j].x - mean, d1 = u[j].y - mean, d2 = u[j].z - mean, d3 = u[j].w - mean;
            ss = fmaf(d0, d0, ss); ss = fmaf(d1, d1, ss); ss = fmaf(d2, d2, ss); ss = fmaf(d3, d3, ss);
        }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
#pragma unroll
    for (int j = 0; j < SW_VEC; j++) {
        const int i = (tid + j * SW_THREADS) * 4;
        if (i < n) {
            const float4 w4 = *reinterpret_cast<const float4*>(wn + i), b4 = *reinterpret_cast<const float4*>(bn + i);
            sw_store4<T>(xn + i, fmaf((u[j].x - mean) * inv, w4.x, b4.x), fmaf((u[j].y - mean) * inv, w4.y, b4.y),
                         fmaf((u[j].z - mean) * inv, w4.z, b4.z), fmaf((u[j].w - mean) * inv, w4.w, b4.w));
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(SW_THREADS) sandwich_step_kernel(float* __restrict__ x, float* __restrict__ y, const float* __restrict__ wp,
                                                                   const float* __restrict__ bp, const float* __restrict__ wn,
                                                                   const float* __restrict__ bn, T* __restrict__ xn, int n, float eps, int vec) {
    __shared__ float scratch[32];
    dependency_wait();
    let_dependents_start();
    const size_t base = (size_t)blockIdx.x * n;
    const int tid = threadIdx.x;
    if (vec) {
        sandwich_row_vec<T>(x + base, y ? y + base : nullptr, wp, bp, wn, bn, xn ? xn + base : nullptr, n, eps, scratch);
        return;
    }
    float v[SW_KEEP];
    if (wp) {
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < SW_KEEP; j++) {
            const int i = tid + j * SW_THREADS;
            v[j] = i < n ? y[base + i] : 0.0f;
            sum += v[j];
        }
        for (int i = tid + SW_KEEP * SW_THREADS; i < n; i += SW_THREADS) sum += y[base + i];
        const float mean = block_sum(sum, scratch) / (float)n;
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < SW_KEEP; j++) {
            const int i = tid + j * SW_THREADS;
            if (i < n) { const float d = v[j] - mean; ss = fmaf(d, d, ss); }
        }
        for (int i = tid + SW_KEEP * SW_THREADS; i < n; i += SW_THREADS) { const float d = y[base + i] - mean; ss = fmaf(d, d, ss); }
        const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
#pragma unroll
        for (int j = 0; j < SW_KEEP; j++) {
            const int i = tid + j * SW_THREADS;
            if (i < n) {
                v[j] = x[base + i] + fmaf((v[j] - mean) * inv, wp[i], bp[i]);
                x[base + i] = v[j];
                y[base + i] = 0.0f;
            }
        }
        for (int i = tid + SW_KEEP * SW_THREADS; i < n; i += SW_THREADS) {
            x[base + i] += fmaf((y[base + i] - mean) * inv, wp[i], bp[i]);
            y[base + i] = 0.0f;
        }
    } else {
#pragma unroll
        for (int j = 0; j < SW_KEEP; j++) {
            const int i = tid + j * SW_THREADS;
            v[j] = i < n ? x[base + i] : 0.0f;
            if (y && i < n) y[base + i] = 0.0f;
        }
        if (y) for (int i = tid + SW_KEEP * SW_THREADS; i < n; i += SW_THREADS) y[base + i] = 0.0f;
    }
    if (!wn) return;
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < SW_KEEP; j++) sum += (tid + j * SW_THREADS < n) ? v[j] : 0.0f;
    for (int i = tid + SW_KEEP * SW_THREADS; i < n; i += SW_THREADS) sum += x[base + i];
    const float mean = block_sum(sum, scratch) / (float)n;
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < SW_KEEP; j++)
        if (tid + j * SW_THREADS < n) { const float d = v[j] - mean; ss = fmaf(d, d, ss); }
    for (int i = tid + SW_KEEP * SW_THREADS; i < n; i += SW_THREADS) { const float d = x[base + i] - mean; ss = fmaf(d, d, ss); }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
#pragma unroll
    for (int j = 0; j < SW_KEEP; j++) {
        const int i = tid + j * SW_THREADS;
        if (i < n) xn[base + i] = from_f32<T>(fmaf((v[j] - mean) * inv, wn[i], bn[i]));
    }
    for (int i = tid + SW_KEEP * SW_THREADS; i < n; i += SW_THREADS) xn[base + i] = from_f32<T>(fmaf((x[base + i] - mean) * inv, wn[i], bn[i]));
}

template <typename T>
__global__ void __launch_bounds__(256) glu_clamped_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, float limit, float alpha) {
    dependency_wait();
    let_dependents_start();
    const T* row = gu + (size_t)blockIdx.x * 2 * inter;
    for (int i = threadIdx.x; i < inter; i += blockDim.x) {
        const float g = fminf(to_f32<T>(row[i]), limit);
        const float u = fminf(fmaxf(to_f32<T>(row[inter + i]), -limit), limit);
        out[(size_t)blockIdx.x * inter + i] = from_f32<T>((g / (1.0f + expf(-alpha * g))) * (u + 1.0f));
    }
}

}  // namespace vk

using namespace vk;

// table [vocab][hidden], second [buckets + 1][hidden] (null: no second row) in dtype; last_token int32 [slots] (may be null when
// second is null); x float32 [tokens][hidden]; xc [tokens][hidden] in dtype or null.
VK_API int vk_embed_hashed(const void* table, const void* second, const int32_t* ids, const int32_t* positions, const int32_t* token_seg,
                           const int32_t* seg_starts, const int32_t* seg_slots, int32_t* last_token, float* x, void* xc, int tokens, int hidden,
                           int vocab, int buckets, int mul_prev, int mul_cur, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (hidden <= 0 || vocab <= 0 || (second && (buckets <= 0 || !last_token))) return VK_BAD_SHAPE;
    if (dtype == 0)
        return launch_dependent(embed_hashed_kernel<float>, dim3(tokens), dim3(256), 0, stream, (const float*)table, (const float*)second, ids,
                                positions, token_seg, seg_starts, seg_slots, last_token, x, (float*)xc, hidden, vocab, buckets, mul_prev, mul_cur);
    return launch_dependent(embed_hashed_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, (const __nv_bfloat16*)table,
                            (const __nv_bfloat16*)second, ids, positions, token_seg, seg_starts, seg_slots, last_token, x, (__nv_bfloat16*)xc,
                            hidden, vocab, buckets, mul_prev, mul_cur);
}

// x, y float32 [rows][n]; w float32 [n]; xc [rows][n] in dtype, or null.
VK_API int vk_residual_norm_step(float* x, float* y, const float* w, void* xc, int rows, int n, float eps, float mult, int dtype,
                                 cudaStream_t stream) {
    if (rows <= 0) return VK_OK;
    if (n <= 0 || (w && !y)) return VK_BAD_SHAPE;
    const int threads = n >= 1024 ? 256 : 128;
    if (dtype == 0)
        return launch_dependent(residual_norm_step_kernel<float>, dim3(rows), dim3(threads), 0, stream, x, y, w, (float*)xc, n, eps, mult);
    return launch_dependent(residual_norm_step_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, x, y, w, (__nv_bfloat16*)xc, n, eps, mult);
}

VK_API int vk_glu_clamped(const void* gu, void* out, int tokens, int inter, float limit, float alpha, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (inter <= 0 || !(limit > 0.0f)) return VK_BAD_SHAPE;
    if (dtype == 0) return launch_dependent(glu_clamped_kernel<float>, dim3(tokens), dim3(256), 0, stream, (const float*)gu, (float*)out, inter, limit, alpha);
    return launch_dependent(glu_clamped_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter,
                            limit, alpha);
}

// x, y float32 [rows][n]; w_post, b_post float32 [n] (both null: nothing is added); w_next, b_next float32 [n] and xn [rows][n] in dtype
// (all null: no normed output).
VK_API int vk_sandwich_step(float* x, float* y, const float* w_post, const float* b_post, const float* w_next, const float* b_next, void* xn, int rows,
                            int n, float eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return VK_OK;
    if (n <= 0 || (w_post && (!y || !b_post)) || (w_next && (!b_next || !xn))) return VK_BAD_SHAPE;
    auto on16 = [](const void* p) { return ((uintptr_t)p % 16) == 0; };
    const int vec = (n % 4 == 0 && n <= 4 * SW_THREADS * SW_VEC && on16(x) && on16(y) && on16(w_post) && on16(b_post) && on16(w_next) && on16(b_next) &&
                     ((uintptr_t)xn % (dtype == 0 ? 16 : 8)) == 0) ? 1 : 0;
    if (dtype == 0)
        return launch_dependent(sandwich_step_kernel<float>, dim3(rows), dim3(SW_THREADS), 0, stream, x, y, w_post, b_post, w_next, b_next, (float*)xn, n, eps,
                                vec);
    return launch_dependent(sandwich_step_kernel<__nv_bfloat16>, dim3(rows), dim3(SW_THREADS), 0, stream, x, y, w_post, b_post, w_next, b_next,
                            (__nv_bfloat16*)xn, n, eps, vec);
}
