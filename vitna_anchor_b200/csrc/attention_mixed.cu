// Attention whose heads' scores are capped and mixed before the softmax, over the paged cache, with rotated values.
//
//  q, k per head: x / rms(x) * w (one weight for all heads; eps < 0: no norm), then the first `dims` values turned in pairs
//                 (i, i + dims/2) by p * f_i (f from the host, any rescaling already in it)
//  v_j            turned over all its pairs (m, m + vdim/2) by j * g_m before it is cached (g null: cached as it is)
//  z_h(i, j)      = scale q_h(i) . k(j), then cap * tanh(z / cap) (cap <= 0: none), then z'_h = sum_g M[h][g] z_g (M null: none)
//  p_h(i, .)      = softmax of z'_h over the keys j <= i (inside the window, if there is one)
//  o_h(i)         = sum_j p_h(i, j) v_j, turned back by -i * g_m
//
//  mixed_attn_prepare   one block a token, a warp a head: from the float32 row of the first product [ q | k | v ] to q in the compute
//                       dtype and k, v in the token's cache slot.
//  attention_mixed_rows one block a query token, all heads: keys in runs of 128 at absolute positions (a thread a key for the scores,
//                       a warp a head for the softmax's running maximum and sum, a thread some (head, value) pairs for the
//                       weighted sum), so the order of an output's sums depends on its own position alone.  Any sizes, both storage
//                       types, prompts' tokens and decoded ones alike.
//
// A page of the cache layer is [nkv][page_size][hd] keys followed by [nkv][page_size][vd] values.  Scores, the cap, the mix,
// the softmax, angles, cos and sin are float32 with accurate tanhf, expf, cosf, sinf.
#include "common.cuh"

namespace vk {

constexpr int AM_THREADS = 128;
constexpr int AM_MAX_ACC = 32;      // (head, value) pairs a thread keeps: heads * vd <= 128 * 32

template <typename T>
__global__ void __launch_bounds__(256) mixed_attn_prepare_kernel(const float* __restrict__ proj, int N, const int32_t* __restrict__ positions,
                                                                 const int32_t* __restrict__ slot, const float* __restrict__ qn_w,
                                                                 const float* __restrict__ kn_w, float eps, const float* __restrict__ freq, int dims,
                                                                 const float* __restrict__ vfreq, T* __restrict__ q_out, T* __restrict__ cache,
                                                                 int nh, int nkv, int hd, int vd, int page_size) {
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const float* in = proj + (size_t)t * N;
    const int s = (slot && cache) ? slot[t] : -1;
    const size_t page_stride = (size_t)nkv * page_size * (hd + vd);
    T* kbase = s >= 0 ? cache + (size_t)(s / page_size) * page_stride : nullptr;
    T* vbase = s >= 0 ? kbase + (size_t)nkv * page_size * hd : nullptr;
    const int off = s >= 0 ? s % page_size : 0;
    const float pos = (float)positions[t];
    const int half = dims / 2, vhalf = vd / 2;
    for (int h = warp; h < nh + 2 * nkv; h += nwarps) {
        if (h < nh + nkv) {                             // a query or key head: norm, weight, rotation
            const float* v = in + (size_t)h * hd;
            const float* w = h < nh ? qn_w : kn_w;
            T* dst = h < nh ? q_out + ((size_t)t * nh + h) * hd : (s >= 0 ? kbase + ((size_t)(h - nh) * page_size + off) * hd : nullptr);
            if (!dst) continue;
            float inv = 1.0f;
            if (eps >= 0.0f) {
                float ss = 0.0f;
                for (int d = lane; d < hd; d += 32) ss = fmaf(v[d], v[d], ss);
                ss = warp_sum(ss);
                inv = 1.0f / sqrtf(ss / (float)hd + eps);
            }
            for (int i = lane; i < half; i += 32) {
                const float ang = pos * freq[i];
                const float c = cosf(ang), sn = sinf(ang);
                const float a = (v[i] * inv) * (w ? w[i] : 1.0f), b = (v[i + half] * inv) * (w ? w[i + half] : 1.0f);
                dst[i] = from_f32<T>(a * c - b * sn);
                dst[i + half] = from_f32<T>(b * c + a * sn);
            }
            for (int d = dims + lane; d < hd; d += 32) dst[d] = from_f32<T>((v[d] * inv) * (w ? w[d] : 1.0f));
        } else if (s >= 0) {                            // a value head
            const int g = h - nh - nkv;
            const float* v = in + (size_t)(nh + nkv) * hd + (size_t)g * vd;
            T* dst = vbase + ((size_t)g * page_size + off) * vd;
            if (vfreq) {
                for (int i = lane; i < vhalf; i += 32) {
                    const float ang = pos * vfreq[i];
                    const float c = cosf(ang), sn = sinf(ang);
                    const float a = v[i], b = v[i + vhalf];
                    dst[i] = from_f32<T>(a * c - b * sn);
                    dst[i + vhalf] = from_f32<T>(b * c + a * sn);
                }
                if (vd & 1) { if (lane == 0) dst[vd - 1] = from_f32<T>(v[vd - 1]); }
            } else {
                for (int d = lane; d < vd; d += 32) dst[d] = from_f32<T>(v[d]);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(AM_THREADS) attention_mixed_rows_kernel(
    const T* __restrict__ q, const T* __restrict__ cache, const int32_t* __restrict__ block_tables, const int32_t* __restrict__ token_seg,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ tok_list, T* __restrict__ out, int nh, int nkv, int hd, int vd,
    int page_size, int max_blocks, float scale, float cap, const float* __restrict__ mix, const float* __restrict__ vfreq, int window) {
    extern __shared__ float am_sh[];
    float* qs = am_sh;                                   // [nh][hd]
    float* raw = qs + (size_t)nh * hd;                   // [nh][128] capped scores, then the outputs [nh][vd] at the end
    float* pr = raw + (size_t)nh * max(AM_THREADS, vd);  // [nh][128] mixed scores, then probabilities
    float* hm = pr + (size_t)nh * AM_THREADS;            // [nh] running maximum
    float* hl = hm + nh;                                 // [nh] running sum
    float* hc = hl + nh;                                 // [nh] this run's correction
    float* mx = hc + nh;                                 // [nh][nh] the mixing matrix
    __shared__ size_t page_off[AM_THREADS];              // element offset of each key's page in the layer's cache
    __shared__ int in_page[AM_THREADS];

    const int t = tok_list ? tok_list[blockIdx.x] : blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = nh / nkv;
    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int32_t* bt = block_tables + (size_t)token_seg[t] * max_blocks;
    const size_t page_stride = (size_t)nkv * page_size * (hd + vd);
    const size_t v_base = (size_t)nkv * page_size * hd;

    const T* qrow = q + (size_t)t * nh * hd;
    for (int i = tid; i < nh * hd; i += AM_THREADS) qs[i] = to_f32<T>(qrow[i]);
    for (int i = tid; i < nh; i += AM_THREADS) { hm[i] = -INFINITY; hl[i] = 0.0f; }
    if (mix) for (int i = tid; i < nh * nh; i += AM_THREADS) mx[i] = mix[i];
    __syncthreads();

    float acc[AM_MAX_ACC];
#pragma unroll
    for (int a = 0; a < AM_MAX_ACC; a++) acc[a] = 0.0f;
    const int n_out = nh * vd;

    for (int c0 = (lo / AM_THREADS) * AM_THREADS; c0 <= pos; c0 += AM_THREADS) {
        const int key = c0 + tid;
        const bool valid = key >= lo && key <= pos;
        if (valid) {
            const int page = bt[key / page_size];
            page_off[tid] = (size_t)page * page_stride;
            in_page[tid] = key % page_size;
            for (int h = 0; h < nh; h++) {
                const T* kr = cache + page_off[tid] + ((size_t)(h / group) * page_size + in_page[tid]) * hd;
                const float* qh = qs + (size_t)h * hd;
                float dot = 0.0f;
                for (int d = 0; d < hd; d++) dot = fmaf(qh[d], to_f32<T>(kr[d]), dot);
                float z = dot * scale;
                if (cap > 0.0f) z = cap * tanhf(z / cap);
                raw[h * AM_THREADS + tid] = z;
            }
            for (int h = 0; h < nh; h++) {
                float z = raw[h * AM_THREADS + tid];
                if (mix) {
                    z = 0.0f;
                    for (int g = 0; g < nh; g++) z = fmaf(mx[h * nh + g], raw[g * AM_THREADS + tid], z);
                }
                pr[h * AM_THREADS + tid] = z;
            }
        } else {
            for (int h = 0; h < nh; h++) pr[h * AM_THREADS + tid] = -INFINITY;
        }
        __syncthreads();
        for (int h = warp; h < nh; h += AM_THREADS / 32) {       // a warp a head: this run's maximum, probabilities and sum
            float* ph = pr + h * AM_THREADS;
            float z[4];
#pragma unroll
            for (int i = 0; i < 4; i++) z[i] = ph[lane + 32 * i];
            const float cmax = warp_max(fmaxf(fmaxf(z[0], z[1]), fmaxf(z[2], z[3])));
            const float m_old = hm[h], m_new = fmaxf(m_old, cmax);
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float p = z[i] == -INFINITY ? 0.0f : expf(z[i] - m_new);
                ph[lane + 32 * i] = p;
                sum += p;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float corr = expf(m_old - m_new);          // 0 on the first run, where m_old is -inf
                hc[h] = corr;
                hl[h] = hl[h] * corr + sum;
                hm[h] = m_new;
            }
        }
        __syncthreads();
        const int j0 = (lo > c0 ? lo : c0) - c0;
        const int j1 = (pos < c0 + AM_THREADS - 1 ? pos : c0 + AM_THREADS - 1) - c0;
#pragma unroll
        for (int a = 0; a < AM_MAX_ACC; a++) {
            const int u = tid + a * AM_THREADS;
            if (u < n_out) {
                const int h = u / vd, d = u - h * vd;
                const size_t head_off = v_base + (size_t)(h / group) * page_size * vd + d;
                const float* ph = pr + h * AM_THREADS;
                float v = acc[a] * hc[h];
                for (int j = j0; j <= j1; j++) v = fmaf(ph[j], to_f32<T>(cache[page_off[j] + head_off + (size_t)in_page[j] * vd]), v);
                acc[a] = v;
            }
        }
        __syncthreads();                                         // the runs' arrays are rewritten by the next run
    }
    // the outputs meet in shared memory, are turned back by the query's position and leave
    float* os = raw;
#pragma unroll
    for (int a = 0; a < AM_MAX_ACC; a++) {
        const int u = tid + a * AM_THREADS;
        if (u < n_out) os[u] = acc[a] / hl[u / vd];
    }
    __syncthreads();
    T* orow = out + (size_t)t * n_out;
    if (vfreq) {
        const int vhalf = vd / 2;
        const float fp = (float)pos;
        for (int u = tid; u < nh * vhalf; u += AM_THREADS) {
            const int h = u / vhalf, i = u - h * vhalf;
            const float ang = fp * vfreq[i];
            const float c = cosf(ang), sn = sinf(ang);
            const float a = os[h * vd + i], b = os[h * vd + i + vhalf];
            orow[h * vd + i] = from_f32<T>(a * c + b * sn);
            orow[h * vd + i + vhalf] = from_f32<T>(b * c - a * sn);
        }
        if (vd & 1) for (int h = tid; h < nh; h += AM_THREADS) orow[h * vd + vd - 1] = from_f32<T>(os[h * vd + vd - 1]);
    } else {
        for (int u = tid; u < n_out; u += AM_THREADS) orow[u] = from_f32<T>(os[u]);
    }
}

}  // namespace vk

using namespace vk;

// proj float32 [tokens][N], N >= nh*hd + nkv*hd + nkv*vd; q_out [tokens][nh*hd] and cache (one layer) in dtype; slot [tokens] or null (-1: no
// write); qn_w, kn_w float32 [hd] or null; eps < 0: no norm; freq float32 [dims/2] (dims 0: no rotation); vfreq float32 [vd/2] or null.
VK_API int vk_mixed_attn_prepare(const float* proj, int N, const int32_t* positions, const int32_t* slot, const float* qn_w, const float* kn_w, float eps,
                                 const float* freq, int dims, const float* vfreq, void* q_out, void* cache, int tokens, int nh, int nkv, int hd, int vd,
                                 int page_size, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (nh <= 0 || nkv <= 0 || hd <= 0 || vd <= 0 || page_size <= 0 || N < (nh + nkv) * hd + nkv * vd || dims < 0 || dims % 2 || dims > hd ||
        (dims > 0 && !freq))
        return VK_BAD_SHAPE;
    if (dtype == 0)
        return launch_dependent(mixed_attn_prepare_kernel<float>, dim3(tokens), dim3(256), 0, stream, proj, N, positions, slot, qn_w, kn_w, eps, freq, dims,
                                vfreq, (float*)q_out, (float*)cache, nh, nkv, hd, vd, page_size);
    return launch_dependent(mixed_attn_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, proj, N, positions, slot, qn_w, kn_w, eps, freq,
                            dims, vfreq, (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, nh, nkv, hd, vd, page_size);
}

VK_API size_t vk_attention_mixed_rows_smem(int nh, int hd, int vd) {
    const size_t runs = (size_t)nh * AM_THREADS, outs = (size_t)nh * vd;
    return ((size_t)nh * hd + (runs > outs ? runs : outs) + runs + 3 * (size_t)nh + (size_t)nh * nh) * sizeof(float);
}

// q [tokens, nh*hd], out [tokens, nh*vd]; cache: one layer [pages][ nkv*page_size*hd keys | nkv*page_size*vd values ]; block_tables
// [segments, max_blocks]; token_seg, positions [all tokens]; tok_list [tokens] names the tokens to run (null: 0..tokens-1); mix float32
// [nh][nh] or null; vfreq float32 [vd/2] or null; cap <= 0: none.
VK_API int vk_attention_mixed_rows(const void* q, const void* cache, const int32_t* block_tables, const int32_t* token_seg, const int32_t* positions,
                                   const int32_t* tok_list, void* out, int tokens, int nh, int nkv, int hd, int vd, int page_size, int max_blocks,
                                   float scale, float cap, const float* mix, const float* vfreq, int window, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || vd <= 0 || page_size <= 0 || max_blocks <= 0 || window < 0) return VK_BAD_SHAPE;
    if ((size_t)nh * vd > (size_t)AM_THREADS * AM_MAX_ACC) return VK_TOO_LARGE;
    const size_t smem = vk_attention_mixed_rows_smem(nh, hd, vd);
    if (smem > 200 * 1024) return VK_TOO_LARGE;
    if (dtype == 0) {
        auto kern = attention_mixed_rows_kernel<float>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<tokens, AM_THREADS, smem, stream>>>((const float*)q, (const float*)cache, block_tables, token_seg, positions, tok_list, (float*)out, nh, nkv,
                                                   hd, vd, page_size, max_blocks, scale, cap, mix, vfreq, window);
    } else {
        auto kern = attention_mixed_rows_kernel<__nv_bfloat16>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<tokens, AM_THREADS, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_tables, token_seg, positions, tok_list,
                                                   (__nv_bfloat16*)out, nh, nkv, hd, vd, page_size, max_blocks, scale, cap, mix, vfreq, window);
    }
    return launch_status();
}
