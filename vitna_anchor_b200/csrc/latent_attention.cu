// The steps of latent attention around its products and the attention itself.
//
// Queries, keys and values pass through narrow latents.  Of a token the cache keeps one row  [ c | kr ]:  the normed
// key-value latent c (kv_rank values) and one rotated key part kr (rot_dim values) that all heads share.  With the keys'
// and values' expansions folded into the neighbouring matrices, a head's query is  [ W_uk^T q_plain | rot(q_rot) ]
// (kv_rank + rot_dim values), its score against a cached row their dot product, and its output the weighted sum of the
// rows' c, which the folded output matrix takes on.  So the attention is one with a single key-value head whose key is the
// row and whose value is the row's first kv_rank values (the attention kernels' "value inside the key" form).  A page of
// the cache layer is [page_size][kv_rank + rot_dim].
//
//  latent_prepare   one block a token, from the float32 row of the first product [ cq_raw | c_raw, kr_raw | ... ]:
//                   cq = cq_raw / rms * w  to the compute dtype;  c = c_raw / rms * w  and  kr = rot(kr_raw, position)  into the
//                   token's cache slot (a layer that reads another layer's cache has no such columns and writes nothing).
//  latent_rotate_q  rotates the last rot_dim values of every head of the query product's result, in place.
//  head_gate        multiplies head h of a token's rows by sigmoid of a float32 column of the first product, in place.
//
// Rotation: pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = (float)p * f_i, cos and sin times
// `mag`; the pairs are (2i, 2i+1) (interleaved) or (i, i + dims/2) of the first `dims` values; f [dims/2] comes from the host
// with any rescaling of the frequencies already in it.  Angles, cos and sin are float32 (accurate cosf and sinf).
#include "common.cuh"

namespace vk {

__device__ __forceinline__ void rot_pair_index(int i, int dims, int interleaved, int& a, int& b) {
    if (interleaved) { a = 2 * i; b = 2 * i + 1; }
    else { a = i; b = i + dims / 2; }
}

template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(
    const float* __restrict__ proj, int N, int q_rank, const float* __restrict__ qn_w, T* __restrict__ cq, int kv_off, int kv_rank,
    int rot_dim, const float* __restrict__ kvn_w, float eps, const int32_t* __restrict__ positions, const float* __restrict__ freq,
    float mag, int dims, int interleaved, const int32_t* __restrict__ slot, T* __restrict__ cache, int page_size) {
    __shared__ float scratch[32];
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* in = proj + (size_t)t * N;
    {
        float ss = 0.0f;
        for (int i = tid; i < q_rank; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
        for (int i = tid; i < q_rank; i += blockDim.x) cq[(size_t)t * q_rank + i] = from_f32<T>((in[i] * inv) * qn_w[i]);
    }
    if (kv_off < 0 || !cache || !slot) return;
    const int s = slot[t];
    if (s < 0) return;                                       // a padding token of a captured batch
    const float* kv = in + kv_off;
    float ss = 0.0f;
    for (int i = tid; i < kv_rank; i += blockDim.x) ss = fmaf(kv[i], kv[i], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)kv_rank + eps);
    const int hd = kv_rank + rot_dim;
    T* krow = cache + (size_t)s * hd;                        // a page is [page_size][hd]: slot s is row s of the layer
    for (int i = tid; i < kv_rank; i += blockDim.x) krow[i] = from_f32<T>((kv[i] * inv) * kvn_w[i]);
    const float* kr = kv + kv_rank;
    const float pos = (float)positions[t];
    for (int i = tid; i < dims / 2; i += blockDim.x) {
        int a, b;
        rot_pair_index(i, dims, interleaved, a, b);
        const float ang = pos * freq[i];
        const float c = cosf(ang) * mag, sn = sinf(ang) * mag;
        const float u = kr[a], v = kr[b];
        krow[kv_rank + a] = from_f32<T>(u * c - v * sn);
        krow[kv_rank + b] = from_f32<T>(v * c + u * sn);
    }
    for (int i = dims + tid; i < rot_dim; i += blockDim.x) krow[kv_rank + i] = from_f32<T>(kr[i]);
}

// q [tokens][H][lat + rot_dim] in place; a thread a pair.
template <typename T>
__global__ void __launch_bounds__(256) latent_rotate_q_kernel(T* __restrict__ q, const int32_t* __restrict__ positions,
                                                              const float* __restrict__ freq, float mag, int H, int lat, int rot_dim, int dims,
                                                              int interleaved) {
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x, half = dims / 2;
    const float pos = (float)positions[t];
    T* row = q + (size_t)t * H * (lat + rot_dim);
    for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        int a, b;
        rot_pair_index(i, dims, interleaved, a, b);
        T* p = row + (size_t)h * (lat + rot_dim) + lat;
        const float ang = pos * freq[i];
        const float c = cosf(ang) * mag, sn = sinf(ang) * mag;
        const float u = to_f32<T>(p[a]), v = to_f32<T>(p[b]);
        p[a] = from_f32<T>(u * c - v * sn);
        p[b] = from_f32<T>(v * c + u * sn);
    }
}

// x [tokens][H][d] in place, times sigmoid(gates[t * N + off + h])
template <typename T>
__global__ void __launch_bounds__(256) head_gate_kernel(T* __restrict__ x, const float* __restrict__ gates, int N, int off, int H, int d) {
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x;
    T* row = x + (size_t)t * H * d;
    for (int i = threadIdx.x; i < H * d; i += blockDim.x) {
        const float g = 1.0f / (1.0f + expf(-gates[(size_t)t * N + off + i / d]));
        row[i] = from_f32<T>(to_f32<T>(row[i]) * g);
    }
}

// The values' expansion behind the attention, for a gate that acts on every value: out[t][h][d] = (sum_r W[h][r][d] lat[t][h][r]) *
// sigmoid(gate[t][h vd + d]).  W is stored [H][rank][vd], so that neighbouring threads read neighbouring values.  A block takes LX_TOKENS
// tokens of one head (a weight is read once for all of them); a sum runs over the rank in one order whatever the batch.
constexpr int LX_TOKENS = 8;
template <typename T>
__global__ void __launch_bounds__(128) latent_expand_gate_kernel(const T* __restrict__ lat, const T* __restrict__ w, const float* __restrict__ gates, int N,
                                                                 int gate_off, int H, int rank, int vd, T* __restrict__ out, int tokens) {
    extern __shared__ float lx_sh[];                    // [LX_TOKENS][rank]
    dependency_wait();
    let_dependents_start();
    const int h = blockIdx.y, t0 = blockIdx.x * LX_TOKENS, cnt = min(LX_TOKENS, tokens - t0);
    for (int i = threadIdx.x; i < LX_TOKENS * rank; i += blockDim.x) {
        const int t = i / rank, r = i - t * rank;
        lx_sh[i] = t < cnt ? to_f32<T>(lat[((size_t)(t0 + t) * H + h) * rank + r]) : 0.0f;
    }
    __syncthreads();
    const T* wh = w + (size_t)h * rank * vd;
    for (int d = threadIdx.x; d < vd; d += blockDim.x) {
        float acc[LX_TOKENS];
#pragma unroll
        for (int t = 0; t < LX_TOKENS; t++) acc[t] = 0.0f;
        for (int r = 0; r < rank; r++) {
            const float wv = to_f32<T>(wh[(size_t)r * vd + d]);
#pragma unroll
            for (int t = 0; t < LX_TOKENS; t++) acc[t] = fmaf(lx_sh[t * rank + r], wv, acc[t]);
        }
#pragma unroll
        for (int t = 0; t < LX_TOKENS; t++)
            if (t < cnt) {
                float v = acc[t];
                if (gates) v *= 1.0f / (1.0f + expf(-gates[(size_t)(t0 + t) * N + gate_off + h * vd + d]));
                out[((size_t)(t0 + t) * H + h) * vd + d] = from_f32<T>(v);
            }
    }
}

}  // namespace vk

using namespace vk;

// lat [tokens][H][rank], w [H][rank][vd] and out [tokens][H][vd] in dtype; gates float32 [tokens][N] with the gate's values at gate_off
// (null: no gate).
VK_API int vk_latent_expand_gate(const void* lat, const void* w, const float* gates, int N, int gate_off, int H, int rank, int vd, void* out, int tokens,
                                 int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (H <= 0 || rank <= 0 || vd <= 0 || (gates && (gate_off < 0 || gate_off + H * vd > N))) return VK_BAD_SHAPE;
    const size_t smem = (size_t)LX_TOKENS * rank * sizeof(float);
    if (smem > 48 * 1024 || H > 65535) return VK_TOO_LARGE;
    dim3 grid((tokens + LX_TOKENS - 1) / LX_TOKENS, H);
    if (dtype == 0)
        return launch_dependent(latent_expand_gate_kernel<float>, grid, dim3(128), smem, stream, (const float*)lat, (const float*)w, gates, N, gate_off, H,
                                rank, vd, (float*)out, tokens);
    return launch_dependent(latent_expand_gate_kernel<__nv_bfloat16>, grid, dim3(128), smem, stream, (const __nv_bfloat16*)lat, (const __nv_bfloat16*)w,
                            gates, N, gate_off, H, rank, vd, (__nv_bfloat16*)out, tokens);
}

// proj float32 [tokens][N]: columns 0..q_rank-1 the query latent, kv_off.. the key-value latent and the shared key part
// (kv_off < 0: none).  cq [tokens][q_rank] and cache in dtype.  slot [tokens] (-1: no write).
VK_API int vk_latent_prepare(const float* proj, int N, int q_rank, const float* qn_w, void* cq, int kv_off, int kv_rank, int rot_dim,
                             const float* kvn_w, float eps, const int32_t* positions, const float* freq, float mag, int dims, int interleaved,
                             const int32_t* slot, void* cache, int page_size, int tokens, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (q_rank <= 0 || N < q_rank || dims < 0 || dims % 2 || dims > rot_dim) return VK_BAD_SHAPE;
    if (kv_off >= 0 && (kv_rank <= 0 || rot_dim < 0 || kv_off + kv_rank + rot_dim > N || page_size <= 0)) return VK_BAD_SHAPE;
    if (dtype == 0)
        return launch_dependent(latent_prepare_kernel<float>, dim3(tokens), dim3(256), 0, stream, proj, N, q_rank, qn_w, (float*)cq, kv_off, kv_rank,
                                rot_dim, kvn_w, eps, positions, freq, mag, dims, interleaved, slot, (float*)cache, page_size);
    return launch_dependent(latent_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, proj, N, q_rank, qn_w, (__nv_bfloat16*)cq,
                            kv_off, kv_rank, rot_dim, kvn_w, eps, positions, freq, mag, dims, interleaved, slot, (__nv_bfloat16*)cache, page_size);
}

VK_API int vk_latent_rotate_q(void* q, const int32_t* positions, const float* freq, float mag, int tokens, int H, int lat, int rot_dim, int dims,
                              int interleaved, int dtype, cudaStream_t stream) {
    if (tokens <= 0 || dims == 0) return VK_OK;
    if (H <= 0 || lat < 0 || dims < 0 || dims % 2 || dims > rot_dim) return VK_BAD_SHAPE;
    if (dtype == 0)
        return launch_dependent(latent_rotate_q_kernel<float>, dim3(tokens), dim3(256), 0, stream, (float*)q, positions, freq, mag, H, lat, rot_dim, dims,
                                interleaved);
    return launch_dependent(latent_rotate_q_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, (__nv_bfloat16*)q, positions, freq, mag, H, lat,
                            rot_dim, dims, interleaved);
}

VK_API int vk_head_gate(void* x, const float* gates, int N, int off, int tokens, int H, int d, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (H <= 0 || d <= 0 || off < 0 || off + H > N) return VK_BAD_SHAPE;
    if (dtype == 0) return launch_dependent(head_gate_kernel<float>, dim3(tokens), dim3(256), 0, stream, (float*)x, gates, N, off, H, d);
    return launch_dependent(head_gate_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, (__nv_bfloat16*)x, gates, N, off, H, d);
}
