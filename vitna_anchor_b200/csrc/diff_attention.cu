// The steps of differential attention around its products and the attention itself.
//
// A head has TWO score maps over one set of values.  Queries and keys carry 2 * dim values a head, laid out [map 1 | map 2];
// after a softmax attention a map, the head's output is  a1 - lambda a2,  divided by its root mean square and scaled by (1 - diff).
// Run as an ordinary attention with 2H query heads, 2G key heads and G value heads (key heads 2g and 2g + 1 read value head g: the
// attention kernels' "several key heads to a value head" form), between the two steps here.
//
//  diff_attn_prepare  one block a token, from the float32 row of the first product [ q | k | v | gate ] (k and v absent in a layer
//                     that reads another layer's cache):  bias;  a short causal convolution over time a channel (the taps - 1 values
//                     before a step's first token come from the request's state slot);  per head and map the RMS norm with a weight
//                     shared by all of them;  pairs (2i, 2i+1) of the first `dims` values turned by position * f_i;  q to the compute
//                     dtype in the order [key head][map][query head of the group], k and v into the token's cache slot.
//  diff_attn_combine  one block a token:  o = a1 - lambda a2;  o / sqrt(mean(o^2) + eps) * (1 - diff) * sigmoid(gate)  in head order;
//                     the block of a segment's last token moves the convolution's memory on.
//
// The convolution's memory of a slot is float32 [taps - 1][channels], oldest row first, zero when the slot is taken, so that
// positions before the sequence's start read zeros.  All arithmetic is float32 with accurate expf, cosf, sinf, sqrtf and division.
#include "common.cuh"

namespace vk {

// The projected value (bias added) of channel c at step-token index src of a segment that starts at `first` with state slot `slot`.
__device__ __forceinline__ float conv_input(const float* __restrict__ proj, int N, const float* __restrict__ bias, const float* __restrict__ tail,
                                            int taps, int C, int slot, int first, int src, int c) {
    if (src >= first) return proj[(size_t)src * N + c] + (bias ? bias[c] : 0.0f);
    const int back = first - src;                       // 1 .. taps - 1 tokens before the step's first
    if (slot < 0 || !tail) return 0.0f;
    return tail[((size_t)slot * (taps - 1) + (taps - 1 - back)) * C + c];
}

template <typename T>
__global__ void __launch_bounds__(256) diff_attn_prepare_kernel(
    const float* __restrict__ proj, int N, const float* __restrict__ bias, const float* __restrict__ conv_w, int taps,
    const float* __restrict__ tail, const int32_t* __restrict__ token_seg, const int32_t* __restrict__ seg_starts,
    const int32_t* __restrict__ seg_slots, const int32_t* __restrict__ positions, const float* __restrict__ qn_w,
    const float* __restrict__ kn_w, float eps, const float* __restrict__ freq, float mag, int dims, int H, int G, int dim, int vdim,
    int own_kv, const int32_t* __restrict__ slot_map, T* __restrict__ cache, int page_size, T* __restrict__ qout,
    const float* __restrict__ out_bias, float* __restrict__ y, int width) {
    extern __shared__ float buf[];                      // [C] the token's channels after the convolution
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x, tid = threadIdx.x;
    const int seg = token_seg[t];
    const int first = seg_starts[seg], slot = seg_slots[seg];
    const int Cq = H * 2 * dim, Ck = own_kv ? G * 2 * dim : 0, Cv = own_kv ? G * vdim : 0;
    const int C = Cq + Ck + Cv;
    for (int c = tid; c < C; c += blockDim.x) {
        float acc;
        if (conv_w) {
            acc = 0.0f;
            for (int j = 0; j < taps; j++)
                acc = fmaf(conv_w[(size_t)c * taps + j], conv_input(proj, N, bias, tail, taps, C, slot, first, t - (taps - 1) + j, c), acc);
        } else {
            acc = proj[(size_t)t * N + c] + (bias ? bias[c] : 0.0f);
        }
        buf[c] = acc;
    }
    if (out_bias)
        for (int i = tid; i < width; i += blockDim.x) y[(size_t)t * width + i] += out_bias[i];
    __syncthreads();

    const int s = (own_kv && slot_map && cache) ? slot_map[t] : -1;
    const size_t page_stride = (size_t)page_size * (2 * G * dim + G * vdim);
    const int page = s >= 0 ? s / page_size : 0, in_page = s >= 0 ? s % page_size : 0;
    const float pos = (float)positions[t];
    const int lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int R = H / G;
    const int rows = 2 * H + (own_kv ? 2 * G : 0);
    for (int r = warp; r < rows; r += nwarps) {
        const bool is_q = r < 2 * H;
        const float* in = buf + (size_t)r * dim;        // q rows, then k rows, are consecutive runs of dim channels
        const float* w = is_q ? qn_w : kn_w;
        float ss = 0.0f;
        for (int i = lane; i < dim; i += 32) ss = fmaf(in[i], in[i], ss);
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
        T* out;
        if (is_q) {
            const int h = r >> 1, mp = r & 1;
            const int g = h / R, hi = h - g * R;
            out = qout + ((size_t)t * 2 * H + (size_t)(g * 2 + mp) * R + hi) * dim;
        } else {
            if (s < 0) continue;                        // a padding token of a captured batch writes nothing
            const int kvh = r - 2 * H;
            out = cache + (size_t)page * page_stride + ((size_t)kvh * page_size + in_page) * dim;
        }
        for (int i = lane; 2 * i < dim; i += 32) {
            const int a = 2 * i, b = 2 * i + 1;
            float u = (in[a] * inv) * w[a];
            float v = b < dim ? (in[b] * inv) * w[b] : 0.0f;
            if (b < dims) {
                const float ang = pos * freq[i];
                const float c = cosf(ang) * mag, sn = sinf(ang) * mag;
                const float ru = u * c - v * sn, rv = v * c + u * sn;
                u = ru; v = rv;
            }
            out[a] = from_f32<T>(u);
            if (b < dim) out[b] = from_f32<T>(v);
        }
    }
    if (s >= 0) {
        const float* vin = buf + Cq + Ck;
        T* vbase = cache + (size_t)page * page_stride + (size_t)2 * G * page_size * dim;
        for (int c = tid; c < Cv; c += blockDim.x) {
            const int g = c / vdim, d = c - g * vdim;
            vbase[((size_t)g * page_size + in_page) * vdim + d] = from_f32<T>(vin[c]);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) diff_attn_combine_kernel(
    const T* __restrict__ att, const float* __restrict__ proj, int N, int gate_off, float lambda, float diff, float eps, int H, int G,
    int vdim, T* __restrict__ out, const float* __restrict__ bias, int taps, int C, float* __restrict__ tail,
    const int32_t* __restrict__ token_seg, const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots) {
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int R = H / G;
    const float keep = 1.0f - diff;
    for (int h = warp; h < H; h += nwarps) {
        const int g = h / R, hi = h - g * R;
        const T* a1 = att + ((size_t)t * 2 * H + (size_t)(g * 2) * R + hi) * vdim;
        const T* a2 = att + ((size_t)t * 2 * H + (size_t)(g * 2 + 1) * R + hi) * vdim;
        float ss = 0.0f;
        for (int d = lane; d < vdim; d += 32) {
            const float o = to_f32<T>(a1[d]) - lambda * to_f32<T>(a2[d]);
            ss = fmaf(o, o, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
        const float* gate = proj + (size_t)t * N + gate_off + (size_t)h * vdim;
        T* orow = out + ((size_t)t * H + h) * vdim;
        for (int d = lane; d < vdim; d += 32) {
            const float o = to_f32<T>(a1[d]) - lambda * to_f32<T>(a2[d]);
            orow[d] = from_f32<T>(((o * inv) * keep) / (1.0f + expf(-gate[d])));
        }
    }
    // the convolution's memory: the last taps - 1 projected values of the request, oldest first
    if (!tail || taps <= 1) return;
    const int seg = token_seg[t];
    const int first = seg_starts[seg], last = seg_starts[seg + 1] - 1, slot = seg_slots[seg];
    if (t != last || slot < 0) return;
    const int n = last - first + 1, keepn = taps - 1;
    float* mine = tail + (size_t)slot * keepn * C;
    for (int c = tid; c < C; c += blockDim.x) {
        for (int r = 0; r < keepn; r++) {              // new row r is the token keepn - 1 - r before the last
            const int src = last - (keepn - 1) + r;
            float v;
            if (src >= first) v = proj[(size_t)src * N + c] + (bias ? bias[c] : 0.0f);
            else v = mine[(size_t)(r + n) * C + c];    // an older row, further down: read before any write reaches it
            mine[(size_t)r * C + c] = v;
        }
    }
}

}  // namespace vk

using namespace vk;

// proj float32 [tokens][N]: columns q [H 2 dim] | k [G 2 dim] | v [G vdim] (the last two only with own_kv) | ...;  bias float32 [>= C] or null;
// conv_w float32 [C][taps] or null (no convolution);  tail float32 [slots][taps - 1][C];  qout [tokens][2H][dim] and cache in dtype;
// cache: one layer [pages][ 2G page_size dim keys | G page_size vdim values ];  out_bias float32 [width] or null is added into y.
VK_API int vk_diff_attn_prepare(const float* proj, int N, const float* bias, const float* conv_w, int taps, const float* tail,
                                const int32_t* token_seg, const int32_t* seg_starts, const int32_t* seg_slots, const int32_t* positions,
                                const float* qn_w, const float* kn_w, float eps, const float* freq, float mag, int dims, int H, int G, int dim,
                                int vdim, int own_kv, const int32_t* slot_map, void* cache, int page_size, void* qout, const float* out_bias,
                                float* y, int width, int tokens, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 || taps < 1 || dims < 0 || dims % 2 || dims > dim) return VK_BAD_SHAPE;
    const int C = H * 2 * dim + (own_kv ? G * 2 * dim + G * vdim : 0);
    if (N < C || (own_kv && page_size <= 0) || (conv_w && taps > 1 && !tail)) return VK_BAD_SHAPE;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 200 * 1024) return VK_TOO_LARGE;
    if (dtype == 0) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(diff_attn_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_dependent(diff_attn_prepare_kernel<float>, dim3(tokens), dim3(256), smem, stream, proj, N, bias, conv_w, taps, tail, token_seg,
                                seg_starts, seg_slots, positions, qn_w, kn_w, eps, freq, mag, dims, H, G, dim, vdim, own_kv, slot_map, (float*)cache,
                                page_size, (float*)qout, out_bias, y, width);
    }
    if (smem > 48 * 1024) cudaFuncSetAttribute(diff_attn_prepare_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(diff_attn_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), smem, stream, proj, N, bias, conv_w, taps, tail,
                            token_seg, seg_starts, seg_slots, positions, qn_w, kn_w, eps, freq, mag, dims, H, G, dim, vdim, own_kv, slot_map,
                            (__nv_bfloat16*)cache, page_size, (__nv_bfloat16*)qout, out_bias, y, width);
}

// att [tokens][2H][vdim] in the order [key head][map][query head of the group], out [tokens][H vdim] in dtype; the gate's columns
// start at gate_off of proj.  tail (or null) as above, C its channels.
VK_API int vk_diff_attn_combine(const void* att, const float* proj, int N, int gate_off, float lambda, float diff, float eps, int H, int G, int vdim,
                                void* out, const float* bias, int taps, int C, float* tail, const int32_t* token_seg, const int32_t* seg_starts,
                                const int32_t* seg_slots, int tokens, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (H <= 0 || G <= 0 || H % G || vdim <= 0 || gate_off < 0 || gate_off + H * vdim > N || taps < 1 || C > N) return VK_BAD_SHAPE;
    if (dtype == 0)
        return launch_dependent(diff_attn_combine_kernel<float>, dim3(tokens), dim3(256), 0, stream, (const float*)att, proj, N, gate_off, lambda, diff,
                                eps, H, G, vdim, (float*)out, bias, taps, C, tail, token_seg, seg_starts, seg_slots);
    return launch_dependent(diff_attn_combine_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, (const __nv_bfloat16*)att, proj, N, gate_off,
                            lambda, diff, eps, H, G, vdim, (__nv_bfloat16*)out, bias, taps, C, tail, token_seg, seg_starts, seg_slots);
}
