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

// PARTIAL: the block takes the runs  blockIdx.y * runs_per_split ..  of its token's keys alone and leaves, instead of the output,
// the unnormalised sums, the maximum and the sum of the weights of every head in part [token][split][nh * (vd + 2)]
// (attention_mixed_combine adds the splits up): single decoded tokens far into a context are spread over many blocks.
template <typename T, bool PARTIAL>
__global__ void __launch_bounds__(AM_THREADS) attention_mixed_rows_kernel(
    const T* __restrict__ q, const T* __restrict__ cache, const int32_t* __restrict__ block_tables, const int32_t* __restrict__ token_seg,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ tok_list, T* __restrict__ out, int nh, int nkv, int hd, int vd,
    int page_size, int max_blocks, float scale, float cap, const float* __restrict__ mix, const float* __restrict__ vfreq, int window,
    float* __restrict__ part, int runs_per_split) {
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

    int c_first = (lo / AM_THREADS) * AM_THREADS, c_last = pos;
    const int n_out = nh * vd;
    if (PARTIAL) {
        c_first = max(c_first, (int)blockIdx.y * runs_per_split * AM_THREADS);
        c_last = min(c_last, ((int)blockIdx.y + 1) * runs_per_split * AM_THREADS - 1);
        if (c_first > c_last) {                                  // no key of this token falls into the split
            float* p = part + ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * (size_t)(n_out + 2 * nh);
            for (int i = tid; i < nh; i += AM_THREADS) { p[n_out + i] = -INFINITY; p[n_out + nh + i] = 0.0f; }
            return;
        }
    }
    const T* qrow = q + (size_t)t * nh * hd;
    for (int i = tid; i < nh * hd; i += AM_THREADS) qs[i] = to_f32<T>(qrow[i]);
    for (int i = tid; i < nh; i += AM_THREADS) { hm[i] = -INFINITY; hl[i] = 0.0f; }
    if (mix) for (int i = tid; i < nh * nh; i += AM_THREADS) mx[i] = mix[i];
    __syncthreads();

    float acc[AM_MAX_ACC];
#pragma unroll
    for (int a = 0; a < AM_MAX_ACC; a++) acc[a] = 0.0f;
    const bool vec = hd % Vec16<T>::N == 0 && (reinterpret_cast<uintptr_t>(cache) % 16 == 0);

    for (int c0 = c_first; c0 <= c_last; c0 += AM_THREADS) {
        const int key = c0 + tid;
        const bool valid = key >= lo && key <= pos;
        if (valid) {
            const int page = bt[key / page_size];
            page_off[tid] = (size_t)page * page_stride;
            in_page[tid] = key % page_size;
            for (int h0 = 0; h0 < nh; h0 += 4) {                // up to four heads of one key-value head share the key's loads
                const int g = h0 / group, hn = min(4, min(nh, (g + 1) * group) - h0);
                const T* kr = cache + page_off[tid] + ((size_t)g * page_size + in_page[tid]) * hd;
                const float* qh = qs + (size_t)h0 * hd;
                float dot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                if (vec) {
                    constexpr int V = Vec16<T>::N;
                    for (int d = 0; d < hd; d += V) {
                        float kv[V];
                        load16<T>(kr + d, kv);
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            if (j < hn) {
#pragma unroll
                                for (int e = 0; e < V; e++) dot[j] = fmaf(qh[j * hd + d + e], kv[e], dot[j]);
                            }
                    }
                } else {
                    for (int d = 0; d < hd; d++) {
                        const float kv = to_f32<T>(kr[d]);
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            if (j < hn) dot[j] = fmaf(qh[j * hd + d], kv, dot[j]);
                    }
                }
                for (int j = 0; j < hn; j++) {
                    float z = dot[j] * scale;
                    if (cap > 0.0f) z = cap * tanhf(z / cap);
                    raw[(h0 + j) * AM_THREADS + tid] = z;
                }
                if (hn < 4) h0 -= 4 - hn;                       // the next group starts where this one ended
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
    if (PARTIAL) {
        float* p = part + ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * (size_t)(n_out + 2 * nh);
#pragma unroll
        for (int a = 0; a < AM_MAX_ACC; a++) {
            const int u = tid + a * AM_THREADS;
            if (u < n_out) p[u] = acc[a];
        }
        for (int i = tid; i < nh; i += AM_THREADS) { p[n_out + i] = hm[i]; p[n_out + nh + i] = hl[i]; }
        return;
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

// Adds up the splits of attention_mixed_rows<PARTIAL>: one block a token.
template <typename T>
__global__ void __launch_bounds__(AM_THREADS) attention_mixed_combine_kernel(const float* __restrict__ part, int nsplit, const int32_t* __restrict__ positions,
                                                                            const int32_t* __restrict__ tok_list, T* __restrict__ out, int nh, int vd,
                                                                            const float* __restrict__ vfreq) {
    extern __shared__ float cb_sh[];                     // [nh][vd] outputs | [nh][nsplit] weights of the splits
    float* os = cb_sh;
    float* wt = cb_sh + (size_t)nh * vd;
    dependency_wait();
    let_dependents_start();
    const int t = tok_list ? tok_list[blockIdx.x] : blockIdx.x, tid = threadIdx.x;
    const int n_out = nh * vd, stride = n_out + 2 * nh;
    const float* base = part + (size_t)blockIdx.x * nsplit * stride;
    for (int h = tid; h < nh; h += AM_THREADS) {         // a split's weight: e^(m_s - M) / sum_s l_s e^(m_s - M)
        float M = -INFINITY;
        for (int s = 0; s < nsplit; s++) M = fmaxf(M, base[(size_t)s * stride + n_out + h]);
        float L = 0.0f;
        for (int s = 0; s < nsplit; s++) {
            const float m = base[(size_t)s * stride + n_out + h];
            const float e = m == -INFINITY ? 0.0f : expf(m - M);
            wt[h * nsplit + s] = e;
            L = fmaf(base[(size_t)s * stride + n_out + nh + h], e, L);
        }
        const float inv = 1.0f / L;
        for (int s = 0; s < nsplit; s++) wt[h * nsplit + s] *= inv;
    }
    __syncthreads();
    for (int u = tid; u < n_out; u += AM_THREADS) {
        const float* w = wt + (u / vd) * nsplit;
        float v = 0.0f;
        for (int s = 0; s < nsplit; s++)
            if (w[s] != 0.0f) v = fmaf(base[(size_t)s * stride + u], w[s], v);      // a split without keys left nothing to read
        os[u] = v;
    }
    __syncthreads();
    T* orow = out + (size_t)t * n_out;
    if (vfreq) {
        const int vhalf = vd / 2;
        const float fp = (float)positions[t];
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

// ---------------------------------------------------------------------------------------------------------------
// Prompt portions on the tensor cores (bfloat16): a block takes 16 query tokens of one segment and ALL heads, a warp a head.
//
// Keys come in steps of 64 at absolute positions.  For a step every warp makes its head's 16 x 64 scores with mma.sync (the
// queries' fragments stay in registers, the keys of the head's key-value head lie in shared memory), caps them and puts them
// into shared memory; after a barrier every warp reads, for its own fragment's places, the scores of all heads and mixes them
// (float32), masks, and carries the running maximum and sum of its 16 rows in registers; the weights leave as two bfloat16
// parts (high and low, so that the product with the values keeps float32 weights' accuracy) and O += P V runs on the tensor
// cores against the values, which lie in shared memory a key a row and are read with transposing loads.  Keys and values of a
// step come by cp.async into one of two stages, the next step's while this step's are worked on.  At the end a thread turns its pairs
// (d, d + vd / 2) back by the query's position: both lie in its own fragment.
// ---------------------------------------------------------------------------------------------------------------

constexpr int MP_ROWS = 16;         // query tokens of a block
constexpr int MP_KEYS = 64;         // keys of a step
constexpr int MP_RAW = MP_KEYS + 4; // floats of a row of capped scores in shared memory

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// the high bfloat16 parts of (x, y) and what they leave, again as bfloat16
__device__ __forceinline__ void split_bf16(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
    __nv_bfloat162 h2, l2;
    h2.x = xh; h2.y = yh;
    l2.x = __float2bfloat16_rn(x - __bfloat162float(xh));
    l2.y = __float2bfloat16_rn(y - __bfloat162float(yh));
    hi = *reinterpret_cast<uint32_t*>(&h2);
    lo = *reinterpret_cast<uint32_t*>(&l2);
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mp_cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// For the bfloat16 tensor-core kernel alone: e^x and tanh(x) through ex2.approx (two units in the last place of a float32) and a fast
// division.  tanh(x) = 1 - 2 / (e^(2x) + 1) is off by about 1e-7 in absolute terms, which the cap's factor turns into a score's error of
// 1e-5 at most, a thousandth of what the bfloat16 queries and keys leave.  The general kernel keeps tanhf and expf.
__device__ __forceinline__ float mp_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float mp_tanh(float x) {
    const float t = mp_exp2(fminf(x, 20.0f) * 2.8853900817779268f);       // e^(2x), the argument bounded so that t stays finite
    return 1.0f - __fdividef(2.0f, t + 1.0f);
}

template <int HD, int VD, int MAXT>       // MAXT: the most threads of a block (32 a head): up to 8 heads leave a thread 255 registers
__global__ void __launch_bounds__(MAXT) attention_mixed_prefill_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache, const int32_t* __restrict__ block_tables,
    const int32_t* __restrict__ tiles, __nv_bfloat16* __restrict__ out, int nh, int nkv, int page_size, int max_blocks, float scale, float cap,
    const float* __restrict__ mix, const float* __restrict__ vfreq, int stages) {
    constexpr int KT = HD / 16, NT = VD / 8, KP = HD + 8, VP = VD + 8;
    extern __shared__ __align__(16) unsigned char mp_sh[];
    const size_t stage_elems = (size_t)nkv * MP_KEYS * (KP + VP);                      // a stage: keys [nkv][64][KP], then values [nkv][64][VP]
    __nv_bfloat16* st0 = reinterpret_cast<__nv_bfloat16*>(mp_sh);
    float* raw = reinterpret_cast<float*>(st0 + (size_t)stages * stage_elems);         // [nh][16][MP_RAW] capped scores
    float* mx = raw + (size_t)nh * MP_ROWS * MP_RAW;                                   // [nh][nh]
    const int tid = threadIdx.x, lane = tid & 31, h = tid >> 5, gid = lane >> 2, tig = lane & 3;
    const int tile = blockIdx.x >> 2, sub = blockIdx.x & 3;
    const int rows = min(MP_ROWS, tiles[tile * 4 + 1] - MP_ROWS * sub);
    if (rows <= 0) return;
    const int t0 = tiles[tile * 4 + 0] + MP_ROWS * sub, pos0 = tiles[tile * 4 + 2] + MP_ROWS * sub, seg = tiles[tile * 4 + 3];
    const int32_t* bt = block_tables + (size_t)seg * max_blocks;
    const int group = nh / nkv, g = h / group;
    const size_t page_stride = (size_t)nkv * page_size * (HD + VD), v_base = (size_t)nkv * page_size * HD;
    if (mix) for (int i = tid; i < nh * nh; i += blockDim.x) mx[i] = mix[i];

    // the head's queries as the 16-row operand: rows gid and gid + 8, per 16 columns two pairs each
    uint32_t qa[KT][4];
    {
        const __nv_bfloat16* q0 = q + ((size_t)(t0 + gid) * nh + h) * HD;
        const __nv_bfloat16* q1 = q + ((size_t)(t0 + gid + 8) * nh + h) * HD;
#pragma unroll
        for (int kt = 0; kt < KT; kt++) {
            qa[kt][0] = gid < rows ? *reinterpret_cast<const uint32_t*>(q0 + kt * 16 + 2 * tig) : 0u;
            qa[kt][1] = gid + 8 < rows ? *reinterpret_cast<const uint32_t*>(q1 + kt * 16 + 2 * tig) : 0u;
            qa[kt][2] = gid < rows ? *reinterpret_cast<const uint32_t*>(q0 + kt * 16 + 8 + 2 * tig) : 0u;
            qa[kt][3] = gid + 8 < rows ? *reinterpret_cast<const uint32_t*>(q1 + kt * 16 + 8 + 2 * tig) : 0u;
        }
    }
    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const int pos_hi = pos0 + rows - 1;
    const int qpos[2] = {pos0 + gid, pos0 + gid + 8};
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;
    constexpr float LOG2E = 1.4426950408889634f;

    // a step's keys and values go from the pages into a stage as they lie (cp.async, 16 bytes a piece); keys beyond the tile's last
    // position are zeros.  With two stages the next step's rows are on their way while this step's are worked on.
    auto issue = [&](int stage, int ks) {
        __nv_bfloat16* Ks = st0 + (size_t)stage * stage_elems;
        __nv_bfloat16* Vs = Ks + (size_t)nkv * MP_KEYS * KP;
        for (int i = tid; i < nkv * MP_KEYS * (HD / 8); i += blockDim.x) {
            const int c = i % (HD / 8), kk = (i / (HD / 8)) % MP_KEYS, gg = i / ((HD / 8) * MP_KEYS);
            const int key = ks + kk;
            __nv_bfloat16* dst = Ks + ((size_t)gg * MP_KEYS + kk) * KP + c * 8;
            if (key <= pos_hi)
                mp_cp16(dst, cache + (size_t)bt[key / page_size] * page_stride + ((size_t)gg * page_size + key % page_size) * HD + c * 8);
            else
                *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
        for (int i = tid; i < nkv * MP_KEYS * (VD / 8); i += blockDim.x) {
            const int c = i % (VD / 8), kk = (i / (VD / 8)) % MP_KEYS, gg = i / ((VD / 8) * MP_KEYS);
            const int key = ks + kk;
            __nv_bfloat16* dst = Vs + ((size_t)gg * MP_KEYS + kk) * VP + c * 8;
            if (key <= pos_hi)
                mp_cp16(dst, cache + (size_t)bt[key / page_size] * page_stride + v_base + ((size_t)gg * page_size + key % page_size) * VD + c * 8);
            else
                *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue(0, 0);
    int step = 0;
    for (int ks = 0; ks <= pos_hi; ks += MP_KEYS, step++) {
        const int stage = stages > 1 ? (step & 1) : 0;
        if (stages > 1 && ks + MP_KEYS <= pos_hi) {
            issue(stage ^ 1, ks + MP_KEYS);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            if (stages == 1 && step > 0) issue(0, ks);                      // one stage: the barrier at the loop's end freed it
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const __nv_bfloat16* Ks = st0 + (size_t)stage * stage_elems;
        const __nv_bfloat16* Vs = Ks + (size_t)nkv * MP_KEYS * KP;
        float s[MP_KEYS / 8][4];
#pragma unroll
        for (int nt = 0; nt < MP_KEYS / 8; nt++) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f; }
        const __nv_bfloat16* kg = Ks + (size_t)g * MP_KEYS * KP;
        // four 8 x 8 pieces a load: keys 8 nt .. and 8 (nt + 1) .., each with columns 16 kt .. + 7 and + 8 .. + 15
        const __nv_bfloat16* k_lane = kg + (size_t)((lane >> 4) * 8 + (lane & 7)) * KP + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int kt = 0; kt < KT; kt++) {
#pragma unroll
            for (int nt = 0; nt < MP_KEYS / 8; nt += 2) {
                uint32_t b[4];
                ldsm_x4(b, k_lane + (size_t)nt * 8 * KP + kt * 16);
                mma_bf16_16816(s[nt], qa[kt], b[0], b[1]);
                mma_bf16_16816(s[nt + 1], qa[kt], b[2], b[3]);
            }
        }
        float* mine = raw + (size_t)h * MP_ROWS * MP_RAW;
#pragma unroll
        for (int nt = 0; nt < MP_KEYS / 8; nt++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float z = s[nt][e] * scale;
                if (cap > 0.0f) z = cap * mp_tanh(z * inv_cap);
                s[nt][e] = z;
            }
            if (mix) {
                *reinterpret_cast<float2*>(mine + gid * MP_RAW + nt * 8 + 2 * tig) = make_float2(s[nt][0], s[nt][1]);
                *reinterpret_cast<float2*>(mine + (gid + 8) * MP_RAW + nt * 8 + 2 * tig) = make_float2(s[nt][2], s[nt][3]);
            }
        }
        if (mix) {
            __syncthreads();
#pragma unroll
            for (int nt = 0; nt < MP_KEYS / 8; nt++) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f; }
            for (int gg = 0; gg < nh; gg++) {
                const float w = mx[h * nh + gg];
                const float* other = raw + (size_t)gg * MP_ROWS * MP_RAW;
#pragma unroll
                for (int nt = 0; nt < MP_KEYS / 8; nt++) {
                    const float2 a = *reinterpret_cast<const float2*>(other + gid * MP_RAW + nt * 8 + 2 * tig);
                    const float2 b = *reinterpret_cast<const float2*>(other + (gid + 8) * MP_RAW + nt * 8 + 2 * tig);
                    s[nt][0] = fmaf(w, a.x, s[nt][0]);
                    s[nt][1] = fmaf(w, a.y, s[nt][1]);
                    s[nt][2] = fmaf(w, b.x, s[nt][2]);
                    s[nt][3] = fmaf(w, b.y, s[nt][3]);
                }
            }
        }
        // mask, this step's maxima, the weights and their sums; rows gid (values 0, 1) and gid + 8 (values 2, 3)
        float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < MP_KEYS / 8; nt++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int key = ks + nt * 8 + 2 * tig + (e & 1);
                if (key > qpos[e >> 1]) s[nt][e] = -INFINITY;
                rmax[e >> 1] = fmaxf(rmax[e >> 1], s[nt][e]);
            }
        }
        float m_use[2], corr[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 1));
            rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 2));
            const float m_new = fmaxf(m_run[r], rmax[r]);
            m_use[r] = m_new == -INFINITY ? 0.0f : m_new;                   // a row of the tile that no token has
            corr[r] = mp_exp2((m_run[r] - m_use[r]) * LOG2E);               // 0 while nothing has been seen
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int nt = 0; nt < MP_KEYS / 8; nt++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float pv = mp_exp2((s[nt][e] - m_use[e >> 1]) * LOG2E);   // 2^(-inf) = 0 for what the mask took
                s[nt][e] = pv;
                l_run[e >> 1] += pv;
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) { o[nt][0] *= corr[0]; o[nt][1] *= corr[0]; o[nt][2] *= corr[1]; o[nt][3] *= corr[1]; }
        // the values lie a key a row: the transposing load gives keys 16 kt .. + 7 and + 8 .. + 15 of columns 8 nt .. and 8 (nt + 1) ..
        const __nv_bfloat16* v_lane = Vs + ((size_t)g * MP_KEYS + (lane & 15)) * VP + (lane >> 4) * 8;
#pragma unroll
        for (int kt = 0; kt < MP_KEYS / 16; kt++) {
            uint32_t hi[4], lo[4];
            split_bf16(s[2 * kt][0], s[2 * kt][1], hi[0], lo[0]);
            split_bf16(s[2 * kt][2], s[2 * kt][3], hi[1], lo[1]);
            split_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1], hi[2], lo[2]);
            split_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3], hi[3], lo[3]);
#pragma unroll
            for (int nt = 0; nt < NT; nt += 2) {
                uint32_t b[4];
                ldsm_x4_trans(b, v_lane + (size_t)kt * 16 * VP + nt * 8);
                mma_bf16_16816(o[nt], hi, b[0], b[1]);
                mma_bf16_16816(o[nt], lo, b[0], b[1]);
                mma_bf16_16816(o[nt + 1], hi, b[2], b[3]);
                mma_bf16_16816(o[nt + 1], lo, b[2], b[3]);
            }
        }
        __syncthreads();                                                    // the step's arrays are filled again
    }
    float inv[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        float l = l_run[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        inv[r] = l > 0.0f ? 1.0f / l : 0.0f;
    }
#pragma unroll
    for (int nt = 0; nt < NT / 2; nt++) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int r = e >> 1, row = gid + 8 * r, d = nt * 8 + 2 * tig + (e & 1);
            float a = o[nt][e] * inv[r], b = o[nt + NT / 2][e] * inv[r];
            if (vfreq) {
                const float ang = (float)qpos[r] * vfreq[d];
                const float c = cosf(ang), sn = sinf(ang);
                const float a2 = a * c + b * sn;
                b = b * c - a * sn;
                a = a2;
            }
            o[nt][e] = a;
            o[nt + NT / 2][e] = b;
            (void)row;
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        if (gid < rows)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + gid) * nh + h) * VD + nt * 8 + 2 * tig) = pack_bf16(o[nt][0], o[nt][1]);
        if (gid + 8 < rows)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + gid + 8) * nh + h) * VD + nt * 8 + 2 * tig) = pack_bf16(o[nt][2], o[nt][3]);
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
        auto kern = attention_mixed_rows_kernel<float, false>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<tokens, AM_THREADS, smem, stream>>>((const float*)q, (const float*)cache, block_tables, token_seg, positions, tok_list, (float*)out, nh, nkv,
                                                   hd, vd, page_size, max_blocks, scale, cap, mix, vfreq, window, nullptr, 0);
    } else {
        auto kern = attention_mixed_rows_kernel<__nv_bfloat16, false>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<tokens, AM_THREADS, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_tables, token_seg, positions, tok_list,
                                                   (__nv_bfloat16*)out, nh, nkv, hd, vd, page_size, max_blocks, scale, cap, mix, vfreq, window, nullptr, 0);
    }
    return launch_status();
}

// The same for single decoded tokens far into a context: the keys of a token are cut into `nsplit` splits of runs_per_split runs of
// 128 keys at absolute positions, a block a (token, split), and a second launch adds the splits up.  part: float32
// [tokens][nsplit][nh * (vd + 2)] scratch.  The launch depends on tokens and nsplit alone.
VK_API int vk_attention_mixed_split(const void* q, const void* cache, const int32_t* block_tables, const int32_t* token_seg, const int32_t* positions,
                                    const int32_t* tok_list, void* out, float* part, int tokens, int nsplit, int runs_per_split, int nh, int nkv, int hd,
                                    int vd, int page_size, int max_blocks, float scale, float cap, const float* mix, const float* vfreq, int window,
                                    int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || vd <= 0 || page_size <= 0 || max_blocks <= 0 || window < 0 || nsplit <= 0 ||
        runs_per_split <= 0 || !part)
        return VK_BAD_SHAPE;
    if ((size_t)nh * vd > (size_t)AM_THREADS * AM_MAX_ACC || nsplit > 65535) return VK_TOO_LARGE;
    const size_t smem = vk_attention_mixed_rows_smem(nh, hd, vd);
    const size_t smem2 = ((size_t)nh * vd + (size_t)nh * nsplit) * sizeof(float);
    if (smem > 200 * 1024 || smem2 > 200 * 1024) return VK_TOO_LARGE;
    dim3 grid(tokens, nsplit);
    int st;
    if (dtype == 0) {
        auto kern = attention_mixed_rows_kernel<float, true>;
        auto comb = attention_mixed_combine_kernel<float>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(comb, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
        if (e != cudaSuccess) return (int)e;
        kern<<<grid, AM_THREADS, smem, stream>>>((const float*)q, (const float*)cache, block_tables, token_seg, positions, tok_list, (float*)out, nh, nkv, hd,
                                                 vd, page_size, max_blocks, scale, cap, mix, vfreq, window, part, runs_per_split);
        st = launch_status();
        if (st != VK_OK) return st;
        return launch_dependent(comb, dim3(tokens), dim3(AM_THREADS), smem2, stream, (const float*)part, nsplit, positions, tok_list, (float*)out, nh, vd, vfreq);
    }
    auto kern = attention_mixed_rows_kernel<__nv_bfloat16, true>;
    auto comb = attention_mixed_combine_kernel<__nv_bfloat16>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(comb, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    if (e != cudaSuccess) return (int)e;
    kern<<<grid, AM_THREADS, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_tables, token_seg, positions, tok_list,
                                             (__nv_bfloat16*)out, nh, nkv, hd, vd, page_size, max_blocks, scale, cap, mix, vfreq, window, part, runs_per_split);
    st = launch_status();
    if (st != VK_OK) return st;
    return launch_dependent(comb, dim3(tokens), dim3(AM_THREADS), smem2, stream, (const float*)part, nsplit, positions, tok_list, (__nv_bfloat16*)out, nh, vd,
                            vfreq);
}

// Prompt portions on the tensor cores, bfloat16: tiles int32 [n_tiles][4] = first token, rows (up to 64), position of the first token,
// segment; a block takes 16 of a tile's rows and all heads (a warp a head, so nh <= 16).  Key and value sizes 64 or 128; no window.
VK_API int vk_attention_mixed_prefill(const void* q, const void* cache, const int32_t* block_tables, const int32_t* tiles, void* out, int n_tiles, int nh,
                                      int nkv, int hd, int vd, int page_size, int max_blocks, float scale, float cap, const float* mix, const float* vfreq,
                                      cudaStream_t stream) {
    if (n_tiles <= 0) return VK_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || max_blocks <= 0) return VK_BAD_SHAPE;
    if (nh > 16 || !((hd == 64 || hd == 128) && (vd == 64 || vd == 128))) return VK_BAD_SHAPE;
    if (((uintptr_t)q % 16) || ((uintptr_t)cache % 16) || ((uintptr_t)out % 4)) return VK_BAD_ALIGNMENT;
    const size_t stage = (size_t)nkv * MP_KEYS * (hd + 8 + vd + 8) * 2, rest = (size_t)nh * MP_ROWS * MP_RAW * 4 + (size_t)nh * nh * 4;
    const int stages = 2 * stage + rest <= 220 * 1024 ? 2 : 1;
    const size_t smem = stages * stage + rest;
    if (smem > 220 * 1024) return VK_TOO_LARGE;
#define VK_MP(HDV, VDV)                                                                                                                       \
    do {                                                                                                                                      \
        auto kern = nh <= 8 ? attention_mixed_prefill_kernel<HDV, VDV, 256> : attention_mixed_prefill_kernel<HDV, VDV, 512>;                  \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                                   \
        if (e != cudaSuccess) return (int)e;                                                                                                  \
        kern<<<n_tiles * 4, nh * 32, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_tables, tiles, (__nv_bfloat16*)out, nh, \
                                                     nkv, page_size, max_blocks, scale, cap, mix, vfreq, stages);                             \
        return launch_status();                                                                                                               \
    } while (0)
    if (hd == 64 && vd == 64) VK_MP(64, 64);
    if (hd == 64 && vd == 128) VK_MP(64, 128);
    if (hd == 128 && vd == 64) VK_MP(128, 64);
    VK_MP(128, 128);
#undef VK_MP
}
