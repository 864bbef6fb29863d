// Residual streams joined by hyper-connections, the embedding that feeds them, and plain activations.
//
// Instead of one residual row a token has S rows X_0..X_{S-1} (float32, stored [tokens][S][width]).  A sublayer f
// with weights a [S], M [S][S] (indexed [from][to]), b [S] and an RMS norm w does
//
//     u = sum_i a_i X_i        y = f(rms(u) * w)        X_j <- sum_i M[i][j] X_i + b_j y      (all j at once)
//
// One kernel does what lies between two sublayers: it applies the update of the sublayer that has just run (its y
// is given), and then forms the next sublayer's input from the new rows, norms it and writes it in the compute
// dtype.  Either half may be absent: the first step of a model has no update, the last one no next sublayer but a
// plain sum of the rows.  The sublayer's parts ADD their result into a float32 buffer, so this kernel also leaves y
// zeroed for the next one.  All arithmetic is float32, a row's sum of squares in a fixed tree.
#include "common.cuh"

namespace vk {

constexpr int HC_MAX_STREAMS = 8;        // sixteen cost the kernel three times its time (registers)
constexpr int HC_THREADS = 256;

// One block per token (256 threads; 1,024 for a step of few tokens, where the kernel is as long as its trips to memory and a
// thread should have one column).  smem: u [width].
template <typename T>
__global__ void __launch_bounds__(1024) hyper_step_kernel(
    float* __restrict__ xs, float* __restrict__ y, const float* __restrict__ mix, const float* __restrict__ out_w,
    const float* __restrict__ in_w, const float* __restrict__ norm_w, float eps, T* __restrict__ xn, float* __restrict__ sum_out,
    int streams, int width) {
    extern __shared__ float u_s[];
    __shared__ float scratch[32];
    __shared__ float m_s[HC_MAX_STREAMS * HC_MAX_STREAMS], b_s[HC_MAX_STREAMS], a_s[HC_MAX_STREAMS];
    const int t = blockIdx.x, tid = threadIdx.x;
    if (tid < streams * streams && mix) m_s[tid] = mix[tid];          // weights: no kernel writes them
    if (tid < streams) {
        if (out_w) b_s[tid] = out_w[tid];
        a_s[tid] = in_w ? in_w[tid] : 1.0f;
    }
    dependency_wait();                                                // the rows and y come from the kernels before this one
    let_dependents_start();
    __syncthreads();
    float* row = xs + (size_t)t * streams * width;
    float ss = 0.0f;
    for (int c = tid; c < width; c += blockDim.x) {
        float x[HC_MAX_STREAMS];
#pragma unroll
        for (int i = 0; i < HC_MAX_STREAMS; i++) x[i] = i < streams ? row[(size_t)i * width + c] : 0.0f;
        if (mix) {
            const float yv = y[(size_t)t * width + c];
            float nx[HC_MAX_STREAMS];
#pragma unroll
            for (int j = 0; j < HC_MAX_STREAMS; j++) {
                float v = 0.0f;
                if (j < streams) {
#pragma unroll
                    for (int i = 0; i < HC_MAX_STREAMS; i++)
                        if (i < streams) v = fmaf(m_s[i * streams + j], x[i], v);
                    v = fmaf(b_s[j], yv, v);
                    row[(size_t)j * width + c] = v;
                }
                nx[j] = v;
            }
#pragma unroll
            for (int j = 0; j < HC_MAX_STREAMS; j++) x[j] = nx[j];
        }
        if (y) y[(size_t)t * width + c] = 0.0f;
        float u = 0.0f;
#pragma unroll
        for (int i = 0; i < HC_MAX_STREAMS; i++)
            if (i < streams) u = fmaf(a_s[i], x[i], u);
        if (sum_out) sum_out[(size_t)t * width + c] = u;
        if (xn) {
            u_s[c] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (!xn) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = tid; c < width; c += blockDim.x) xn[(size_t)t * width + c] = from_f32<T>((u_s[c] * inv) * norm_w[c]);
}

// xs[t][j][:] = scale * table[ids[t]][:] + pos_table[positions[t]][:] for every copy j (pos_table may be null).
template <typename T>
__global__ void embed_scaled_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids, const int32_t* __restrict__ positions,
                                    const float* __restrict__ pos_table, float scale, float* __restrict__ xs, int width, int vocab,
                                    int max_positions, int copies) {
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;      // the host has checked the range; never read outside the tables
    int p = positions[t];
    if (p < 0 || p >= max_positions) p = 0;
    const T* row = table + (size_t)id * width;
    const float* prow = pos_table ? pos_table + (size_t)p * width : nullptr;
    float* out = xs + (size_t)t * copies * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = to_f32<T>(row[c]) * scale;
        if (prow) v += prow[c];
        for (int j = 0; j < copies; j++) out[(size_t)j * width + c] = v;
    }
}

// 0: gelu, the erf form  0.5 z (1 + erf(z / sqrt 2));  1: gelu, the tanh form;  2: silu
template <int KIND> __device__ __forceinline__ float activate(float z) {
    if (KIND == 0) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
    if (KIND == 1) return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
    return z / (1.0f + expf(-z));
}

template <typename T, int KIND>
__global__ void activation_kernel(const T* x, T* out, size_t n) {       // out may be x
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(activate<KIND>(to_f32<T>(x[i])));
}

// f(z) = a_pos z^2 + z/2 for z > 0, a_neg (e^z - 1 - z) + z/2 otherwise: an activation with two numbers of its own
template <typename T>
__global__ void xielu_kernel(const T* x, T* out, size_t n, float a_pos, float a_neg) {       // out may be x
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float z = to_f32<T>(x[i]);
        out[i] = from_f32<T>(z > 0.0f ? fmaf(a_pos * z, z, 0.5f * z) : fmaf(a_neg, expm1f(z) - z, 0.5f * z));
    }
}

}  // namespace vk

using namespace vk;

// xs [tokens][streams][width] float32; y [tokens][width] float32 (null only when there is no update and nothing to
// zero); mix [streams][streams] and out_w [streams] (both null: no update); in_w [streams] (null: all ones); norm_w
// [width] and xn [tokens][width] in dtype (both null: no normed output); sum_out [tokens][width] float32 or null.
VK_API int vk_hyper_step(float* xs, float* y, const float* mix, const float* out_w, const float* in_w, const float* norm_w, float eps,
                         void* xn, float* sum_out, int tokens, int streams, int width, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (streams <= 0 || width <= 0 || (mix == nullptr) != (out_w == nullptr) || (xn == nullptr) != (norm_w == nullptr) || (mix && !y))
        return VK_BAD_SHAPE;
    if (streams > HC_MAX_STREAMS || (size_t)width * sizeof(float) > 200 * 1024) return VK_TOO_LARGE;
    const size_t smem = (size_t)width * sizeof(float);
    const int threads = tokens > 64 ? HC_THREADS : (width >= 1024 ? 1024 : (width + 31) / 32 * 32 < HC_THREADS ? HC_THREADS : (width + 31) / 32 * 32);
    if (dtype == 0) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_step_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (tokens > 64)        // a prompt: an ordinary launch (waiting blocks would hold places the kernel before still needs)
            return launch_plain(hyper_step_kernel<float>, dim3(tokens), dim3(threads), smem, stream, xs, y, mix, out_w, in_w, norm_w, eps,
                                (float*)xn, sum_out, streams, width);
        return launch_dependent(hyper_step_kernel<float>, dim3(tokens), dim3(threads), smem, stream, xs, y, mix, out_w, in_w, norm_w, eps,
                                (float*)xn, sum_out, streams, width);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_step_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (tokens > 64)
            return launch_plain(hyper_step_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), smem, stream, xs, y, mix, out_w, in_w, norm_w,
                                eps, (__nv_bfloat16*)xn, sum_out, streams, width);
        return launch_dependent(hyper_step_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), smem, stream, xs, y, mix, out_w, in_w, norm_w,
                                eps, (__nv_bfloat16*)xn, sum_out, streams, width);
    }
}

VK_API int vk_embed_scaled(const void* table, const int32_t* ids, const int32_t* positions, const float* pos_table, float scale, float* xs,
                           int tokens, int width, int vocab, int max_positions, int copies, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (width <= 0 || vocab <= 0 || copies <= 0 || (pos_table && max_positions <= 0)) return VK_BAD_SHAPE;
    if (dtype == 0)
        embed_scaled_kernel<float><<<tokens, 128, 0, stream>>>((const float*)table, ids, positions, pos_table, scale, xs, width, vocab,
                                                                max_positions, copies);
    else
        embed_scaled_kernel<__nv_bfloat16><<<tokens, 128, 0, stream>>>((const __nv_bfloat16*)table, ids, positions, pos_table, scale, xs,
                                                                        width, vocab, max_positions, copies);
    return launch_status();
}

template <typename T>
static int launch_activation(const void* x, void* out, size_t n, int kind, cudaStream_t stream) {
    size_t g = (n + 255) / 256;
    const int grid = (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
    if (kind == 0) activation_kernel<T, 0><<<grid, 256, 0, stream>>>((const T*)x, (T*)out, n);
    else if (kind == 1) activation_kernel<T, 1><<<grid, 256, 0, stream>>>((const T*)x, (T*)out, n);
    else if (kind == 2) activation_kernel<T, 2><<<grid, 256, 0, stream>>>((const T*)x, (T*)out, n);
    else return VK_BAD_SHAPE;
    return launch_status();
}

// out = act(x) element by element (out may be x); kind as above.
VK_API int vk_activation(const void* x, void* out, size_t n, int kind, int dtype, cudaStream_t stream) {
    if (n == 0) return VK_OK;
    return dtype == 0 ? launch_activation<float>(x, out, n, kind, stream) : launch_activation<__nv_bfloat16>(x, out, n, kind, stream);
}

// out = a_pos x^2 + x/2 where x > 0, a_neg (exp(x) - 1 - x) + x/2 elsewhere (out may be x)
VK_API int vk_xielu(const void* x, void* out, size_t n, float a_pos, float a_neg, int dtype, cudaStream_t stream) {
    if (n == 0) return VK_OK;
    size_t g = (n + 255) / 256;
    const int grid = (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
    if (dtype == 0) xielu_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (float*)out, n, a_pos, a_neg);
    else xielu_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n, a_pos, a_neg);
    return launch_status();
}
