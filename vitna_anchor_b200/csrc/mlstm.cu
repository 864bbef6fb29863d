// The matrix memory with exponential gates (mLSTM): a recurrent mixer whose state is, per head, a matrix S [dim][vdim], a vector
// n [dim] and the running maximum m of the gates' logarithms.
//
//  i_t = cap tanh(a_t / cap),  f_t = log sigmoid(cap tanh(b_t / cap))          a, b: the gates' projections with their biases
//  m_t = max(f_t + m_(t-1), i_t)                                               m starts at 0, S and n at zero
//  S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T;   n_t likewise with k_t alone
//  o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6),  q_t scaled by dim^-1/2
//
//  mlstm_recurrence   token after token, one block per (32 value columns, head, segment).  A warp holds 8 columns of S; its lanes are
//                     4 groups of rows (row d belongs to group d mod 4), so a thread keeps dim / 4 values of its column and of n in
//                     registers and a token's sums over the rows end with two shuffles.  The gates and m are worked out by every
//                     thread alike.  Reads the float32 row of the first product [ q | k | v | gate | a | b ]; writes o float32 and,
//                     after the segment's last token, the state.
//  mlstm_gate         one block a token: each head's o divided by its root mean square, times the norm's weight (all heads' size),
//                     times sigmoid(gate), to the compute dtype.
//
// The state of a slot is float32 [ S: H dim vdim | n: H dim | m: H ].  Everything is float32 with accurate expf, tanhf and log1pf, and the
// order of the sums of an output does not depend on how the tokens were cut into steps.
#include "common.cuh"

namespace vk {

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

template <int DPT>
__global__ void __launch_bounds__(128) mlstm_recurrence_kernel(const float* __restrict__ proj, int N, int H, int dim, int vdim,
                                                               const float* __restrict__ gate_bias, float cap, float qscale,
                                                               const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots,
                                                               float* __restrict__ state, size_t state_floats, float* __restrict__ o) {
    dependency_wait();
    let_dependents_start();
    const int seg = blockIdx.z, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rg = lane >> 3;                                       // rows rg, rg + 4, ...
    const int col = blockIdx.x * 32 + warp * 8 + (lane & 7);
    const bool live = col < vdim;
    const int first = seg_starts[seg], end = seg_starts[seg + 1], slot = seg_slots[seg];
    if (first >= end) return;
    float* st = slot >= 0 ? state + (size_t)slot * state_floats : nullptr;
    float* S_st = st ? st + (size_t)h * dim * vdim : nullptr;
    float* n_st = st ? st + (size_t)H * dim * vdim + (size_t)h * dim : nullptr;
    float* m_st = st ? st + (size_t)H * dim * vdim + (size_t)H * dim + h : nullptr;
    float S[DPT], n[DPT];
#pragma unroll
    for (int j = 0; j < DPT; j++) {
        const int d = rg + 4 * j;
        S[j] = (st && live && d < dim) ? S_st[(size_t)d * vdim + col] : 0.0f;
        n[j] = (st && d < dim) ? n_st[d] : 0.0f;
    }
    float m = st ? *m_st : 0.0f;
    const int q_off = h * dim, k_off = H * dim + h * dim, v_off = 2 * H * dim + h * vdim;
    const int i_off = 2 * H * dim + 2 * H * vdim + h, f_off = i_off + H;
    for (int t = first; t < end; t++) {
        const float* row = proj + (size_t)t * N;
        const float ig = cap * tanhf((row[i_off] + gate_bias[h]) / cap);
        const float fg = log_sigmoid(cap * tanhf((row[f_off] + gate_bias[H + h]) / cap));
        const float m_new = fmaxf(fg + m, ig);
        const float a = expf(fg + m - m_new), b = expf(ig - m_new);
        m = m_new;
        const float vv = live ? row[v_off + col] : 0.0f;
        float po = 0.0f, pn = 0.0f;
#pragma unroll
        for (int j = 0; j < DPT; j++) {
            const int d = rg + 4 * j;
            if (d < dim) {
                const float bk = b * row[k_off + d], qd = row[q_off + d] * qscale;
                S[j] = fmaf(a, S[j], bk * vv);
                n[j] = fmaf(a, n[j], bk);
                po = fmaf(S[j], qd, po);
                pn = fmaf(n[j], qd, pn);
            }
        }
        po += __shfl_xor_sync(0xffffffffu, po, 8);
        po += __shfl_xor_sync(0xffffffffu, po, 16);
        pn += __shfl_xor_sync(0xffffffffu, pn, 8);
        pn += __shfl_xor_sync(0xffffffffu, pn, 16);
        if (live && rg == 0) o[(size_t)t * H * vdim + h * vdim + col] = po / (fmaxf(fabsf(pn), expf(-m)) + 1e-6f);
    }
    if (!st) return;
#pragma unroll
    for (int j = 0; j < DPT; j++) {
        const int d = rg + 4 * j;
        if (d < dim) {
            if (live) S_st[(size_t)d * vdim + col] = S[j];
            if (blockIdx.x == 0 && warp == 0 && (lane & 7) == 0) n_st[d] = n[j];
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *m_st = m;
}

template <typename T>
__global__ void __launch_bounds__(256) mlstm_gate_kernel(const float* __restrict__ o, const float* __restrict__ proj, int N, int gate_off,
                                                         const float* __restrict__ w, float eps, int H, int vdim, T* __restrict__ out) {
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int h = warp; h < H; h += nwarps) {
        const float* in = o + ((size_t)t * H + h) * vdim;
        float ss = 0.0f;
        for (int d = lane; d < vdim; d += 32) ss = fmaf(in[d], in[d], ss);
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
        const float* gate = proj + (size_t)t * N + gate_off + (size_t)h * vdim;
        for (int d = lane; d < vdim; d += 32)
            out[((size_t)t * H + h) * vdim + d] = from_f32<T>(((in[d] * inv) * w[h * vdim + d]) / (1.0f + expf(-gate[d])));
    }
}

}  // namespace vk

using namespace vk;

VK_API int vk_mlstm_max_dim() { return 256; }

// proj float32 [tokens][N] = q [H dim] | k [H dim] | v [H vdim] | gate [H vdim] | a [H] | b [H];  gate_bias float32 [2H] (a's, then b's);
// state float32 [slots][H dim vdim + H dim + H];  o float32 [tokens][H vdim].  A block a (32 columns, head, segment): segments is the
// step's count, whatever their lengths.
VK_API int vk_mlstm_recurrence(const float* proj, int N, int H, int dim, int vdim, const float* gate_bias, float cap, const int32_t* seg_starts,
                               const int32_t* seg_slots, float* state, float* o, int segments, cudaStream_t stream) {
    if (segments <= 0) return VK_OK;
    if (H <= 0 || dim <= 0 || vdim <= 0 || !(cap > 0.0f) || N < 2 * H * dim + 2 * H * vdim + 2 * H) return VK_BAD_SHAPE;
    if (dim > 256 || H > 65535 || segments > 65535) return VK_TOO_LARGE;
    const size_t state_floats = (size_t)H * dim * vdim + (size_t)H * dim + H;
    const float qscale = 1.0f / sqrtf((float)dim);
    dim3 grid((vdim + 31) / 32, H, segments);
#define VK_MLSTM(D)                                                                                                                          \
    return launch_dependent(mlstm_recurrence_kernel<D>, grid, dim3(128), 0, stream, proj, N, H, dim, vdim, gate_bias, cap, qscale, seg_starts, \
                            seg_slots, state, state_floats, o)
    if (dim <= 32) VK_MLSTM(8);
    if (dim <= 64) VK_MLSTM(16);
    if (dim <= 128) VK_MLSTM(32);
    VK_MLSTM(64);
#undef VK_MLSTM
}

VK_API int vk_mlstm_gate(const float* o, const float* proj, int N, int gate_off, const float* w, float eps, int H, int vdim, void* out, int tokens,
                         int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (H <= 0 || vdim <= 0 || gate_off < 0 || gate_off + H * vdim > N) return VK_BAD_SHAPE;
    if (dtype == 0) return launch_dependent(mlstm_gate_kernel<float>, dim3(tokens), dim3(256), 0, stream, o, proj, N, gate_off, w, eps, H, vdim, (float*)out);
    return launch_dependent(mlstm_gate_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, o, proj, N, gate_off, w, eps, H, vdim,
                            (__nv_bfloat16*)out);
}
