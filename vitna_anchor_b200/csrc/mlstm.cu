// The matrix memory with exponential gates (mLSTM): a recurrent mixer whose state is, per head, a matrix S [dim][vdim], a vector
// n [dim] and the running maximum m of the gates' logarithms.
//
//  i_t = cap tanh(a_t / cap),  f_t = log sigmoid(cap tanh(b_t / cap))          a, b: the gates' projections with their biases
//  m_t = max(f_t + m_(t-1), i_t)                                               m starts at 0, S and n at zero
//  S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T;   n_t likewise with k_t alone
//  o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6),  q_t scaled by dim^-1/2
//
//  mlstm_recurrence   token after token, one block per (16 columns, head, segment).  The columns of a head are those of S and, as
//                     column number vdim, n itself (n is the column that a value of 1 would fill), so that nobody works n out twice.
//                     A warp holds 4 columns; its lanes are 8 groups of rows (group g has rows 32 j + 4 g .. + 3), so a thread keeps
//                     dim / 8 values of its column in registers, reads keys and queries as float4 and a token's sum over the rows
//                     ends with three shuffles (a head of 256 values is 17 blocks: the chain is latency, and narrow blocks put it
//                     on more multiprocessors).  Tokens come in chunks of 32 (16 for keys of more than 128 values) through a ring of
//                     two stages in shared memory that cp.async fills a chunk ahead: q, k, the block's columns of v and the two
//                     gates' sums.  For a chunk the gates are worked out side by side (tanh, log sigmoid), one thread carries m
//                     through the chunk (an addition and a maximum a token), and the factors e^(f + m' - m) and e^(i - m) side by
//                     side again: a token's step in the chain is multiplications and additions only.  Reads the float32 row of the
//                     first product [ q | k | v | gate | a | b ]; writes, per token and head, the numerators S^T q, then n . q, then
//                     m (float32 [tokens][H][vdim + 2]) and, after the segment's last token, S and n of the state.
//  mlstm_gate         one block a token: o = numerator / (max(|n . q|, e^-m) + 1e-6), each head's o divided by its root mean square,
//                     times the norm's weight (all heads' size), times sigmoid(gate), to the compute dtype.  One more block a
//                     segment puts the m after the segment's last token into the state: no block of the recurrence may, because
//                     another block of the same head may not have read the old one yet.
//
// The state of a slot is float32 [ S: H dim vdim | n: H dim | m: H ].  Everything is float32 with accurate expf, tanhf and log1pf, and the
// order of the sums of an output does not depend on how the tokens were cut into steps.
#include "common.cuh"

namespace vk {

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

constexpr int ML_THREADS = 128;
constexpr int ML_COLS = 16;
constexpr int ML_ROW_GROUPS = 8;

__device__ __forceinline__ void ml_cp4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ml_cp16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// Floats of one stage: q [C][8 DPT] | k [C][8 DPT] | v [C][16] | the gates' sums [C][2]
__host__ __device__ constexpr int ml_stage_floats(int C, int DPT) { return C * (2 * ML_ROW_GROUPS * DPT + ML_COLS + 2); }

template <int DPT, int C>
__global__ void __launch_bounds__(ML_THREADS) mlstm_recurrence_kernel(const float* __restrict__ proj, int N, int H, int dim, int vdim,
                                                                      const float* __restrict__ gate_bias, float cap, float qscale,
                                                                      const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots,
                                                                      float* __restrict__ state, size_t state_floats, float* __restrict__ o, int vec) {
    constexpr int DP = ML_ROW_GROUPS * DPT;                                     // rows of the state as the registers hold them (dim rounded up)
    constexpr int STAGE = ml_stage_floats(C, DPT);
    extern __shared__ __align__(16) float ml_smem[];
    __shared__ float sgi[C], sgf[C], smp[C], smn[C], sa[C], sb[C];
    dependency_wait();
    let_dependents_start();
    const int seg = blockIdx.z, h = blockIdx.y, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int rg = lane >> 2;                                       // rows 32 j + 4 rg .. + 3
    const int cl = warp * 4 + (lane & 3);
    const int col0 = blockIdx.x * ML_COLS, col = col0 + cl;
    const int first = seg_starts[seg], end = seg_starts[seg + 1], slot = seg_slots[seg];
    if (first >= end) return;
    float* st = slot >= 0 ? state + (size_t)slot * state_floats : nullptr;
    // column vdim is n: its rows lie one after another in the state
    float* col_st = !st || col > vdim ? nullptr
                    : col < vdim ? st + (size_t)h * dim * vdim + col : st + (size_t)H * dim * vdim + (size_t)h * dim;
    const size_t col_stride = col < vdim ? (size_t)vdim : 1;
    float S[DPT];
#pragma unroll
    for (int j = 0; j < DPT / 4; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int d = 32 * j + 4 * rg + i;
            S[4 * j + i] = (col_st && d < dim) ? col_st[(size_t)d * col_stride] : 0.0f;
        }
    float m = st ? st[(size_t)H * dim * vdim + (size_t)H * dim + h] : 0.0f;       // (thread 0's copy is the one that is carried)
    const int q_off = h * dim, k_off = H * dim + h * dim, v_off = 2 * H * dim + h * vdim + col0;
    const int i_off = 2 * H * dim + 2 * H * vdim + h, f_off = i_off + H;
    const int v_cnt = min(ML_COLS, vdim - col0);                    // this block's columns of v (none for a block that has n alone)
    const int OW = vdim + 2;
    // what cp.async never writes: rows beyond dim are zero, column vdim reads 1, columns beyond it 0
    for (int s = 0; s < 2; s++) {
        float* sq = ml_smem + s * STAGE;
        float* sk = sq + C * DP;
        float* sv = sk + C * DP;
        for (int e = tid; e < C * DP; e += ML_THREADS)
            if (e % DP >= dim) { sq[e] = 0.0f; sk[e] = 0.0f; }
        for (int e = tid; e < C * ML_COLS; e += ML_THREADS) {
            const int c = col0 + e % ML_COLS;
            if (c >= vdim) sv[e] = c == vdim ? 1.0f : 0.0f;
        }
    }
    auto issue = [&](int chunk) {
        float* sq = ml_smem + (chunk & 1) * STAGE;
        float* sk = sq + C * DP;
        float* sv = sk + C * DP;
        float* sr = sv + C * ML_COLS;
        const int t0 = first + chunk * C, cnt = min(C, end - t0);
        for (int t = warp; t < cnt; t += ML_THREADS / 32) {
            const float* row = proj + (size_t)(t0 + t) * N;
            if (vec) {
                for (int c = 4 * lane; c < dim; c += 128) { ml_cp16(sq + t * DP + c, row + q_off + c); ml_cp16(sk + t * DP + c, row + k_off + c); }
                if (4 * lane < v_cnt) ml_cp16(sv + t * ML_COLS + 4 * lane, row + v_off + 4 * lane);
            } else {
                for (int c = lane; c < dim; c += 32) { ml_cp4(sq + t * DP + c, row + q_off + c); ml_cp4(sk + t * DP + c, row + k_off + c); }
                if (lane < v_cnt) ml_cp4(sv + t * ML_COLS + lane, row + v_off + lane);
            }
            if (lane == 0) { ml_cp4(sr + 2 * t, row + i_off); ml_cp4(sr + 2 * t + 1, row + f_off); }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int chunks = (end - first + C - 1) / C;
    issue(0);
    for (int c = 0; c < chunks; c++) {
        if (c + 1 < chunks) {
            issue(c + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* sq = ml_smem + (c & 1) * STAGE;
        const float* sk = sq + C * DP;
        const float* sv = sk + C * DP;
        const float* sr = sv + C * ML_COLS;
        const int t0 = first + c * C, cnt = min(C, end - t0);
        if (tid < cnt) {
            sgi[tid] = cap * tanhf((sr[2 * tid] + gate_bias[h]) / cap);
            sgf[tid] = log_sigmoid(cap * tanhf((sr[2 * tid + 1] + gate_bias[H + h]) / cap));
        }
        __syncthreads();
        if (tid == 0) {
#pragma unroll
            for (int t = 0; t < C; t++) {
                if (t < cnt) {
                    const float m_new = fmaxf(sgf[t] + m, sgi[t]);
                    smp[t] = m;
                    smn[t] = m_new;
                    m = m_new;
                }
            }
        }
        __syncthreads();
        if (tid < cnt) {
            sa[tid] = expf(sgf[tid] + smp[tid] - smn[tid]);
            sb[tid] = expf(sgi[tid] - smn[tid]);
            if (blockIdx.x == 0) o[((size_t)(t0 + tid) * H + h) * OW + vdim + 1] = smn[tid];
        }
        __syncthreads();
#pragma unroll 4
        for (int t = 0; t < cnt; t++) {
            const float a = sa[t], bv = sb[t] * sv[t * ML_COLS + cl];
            const float4* k4 = reinterpret_cast<const float4*>(sk + t * DP) + rg;
            const float4* q4 = reinterpret_cast<const float4*>(sq + t * DP) + rg;
            float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
            for (int j = 0; j < DPT / 4; j++) {
                const float4 kk = k4[ML_ROW_GROUPS * j], qq = q4[ML_ROW_GROUPS * j];
                S[4 * j + 0] = fmaf(kk.x, bv, a * S[4 * j + 0]);
                S[4 * j + 1] = fmaf(kk.y, bv, a * S[4 * j + 1]);
                S[4 * j + 2] = fmaf(kk.z, bv, a * S[4 * j + 2]);
                S[4 * j + 3] = fmaf(kk.w, bv, a * S[4 * j + 3]);
                p0 = fmaf(S[4 * j + 0], qq.x, p0);
                p1 = fmaf(S[4 * j + 1], qq.y, p1);
                p2 = fmaf(S[4 * j + 2], qq.z, p2);
                p3 = fmaf(S[4 * j + 3], qq.w, p3);
            }
            float po = (p0 + p1) + (p2 + p3);
            po += __shfl_xor_sync(0xffffffffu, po, 4);
            po += __shfl_xor_sync(0xffffffffu, po, 8);
            po += __shfl_xor_sync(0xffffffffu, po, 16);
            if (rg == 0 && col <= vdim) o[((size_t)(t0 + t) * H + h) * OW + col] = po * qscale;
        }
        __syncthreads();                                            // the stage is filled again at the top of the next round
    }
    if (!col_st) return;
#pragma unroll
    for (int j = 0; j < DPT / 4; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int d = 32 * j + 4 * rg + i;
            if (d < dim) col_st[(size_t)d * col_stride] = S[4 * j + i];
        }
}

template <typename T>
__global__ void __launch_bounds__(256) mlstm_gate_kernel(const float* __restrict__ o, const float* __restrict__ proj, int N, int gate_off,
                                                         const float* __restrict__ w, float eps, int H, int dim, int vdim, T* __restrict__ out,
                                                         int tokens, const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots,
                                                         float* __restrict__ state, size_t state_floats) {
    dependency_wait();
    let_dependents_start();
    const int OW = vdim + 2;
    if ((int)blockIdx.x >= tokens) {                     // a segment's block: m after its last token goes into the state
        const int seg = blockIdx.x - tokens;
        const int first = seg_starts[seg], end = seg_starts[seg + 1], slot = seg_slots[seg];
        if (first >= end || slot < 0) return;
        float* m_st = state + (size_t)slot * state_floats + (size_t)H * dim * vdim + (size_t)H * dim;
        for (int h = threadIdx.x; h < H; h += blockDim.x) m_st[h] = o[((size_t)(end - 1) * H + h) * OW + vdim + 1];
        return;
    }
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int h = warp; h < H; h += nwarps) {
        const float* in = o + ((size_t)t * H + h) * OW;
        const float inv_den = 1.0f / (fmaxf(fabsf(in[vdim]), expf(-in[vdim + 1])) + 1e-6f);
        float ss = 0.0f;
        for (int d = lane; d < vdim; d += 32) {
            const float v = in[d] * inv_den;
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
        const float* gate = proj + (size_t)t * N + gate_off + (size_t)h * vdim;
        for (int d = lane; d < vdim; d += 32)
            out[((size_t)t * H + h) * vdim + d] = from_f32<T>((((in[d] * inv_den) * inv) * w[h * vdim + d]) / (1.0f + expf(-gate[d])));
    }
}

}  // namespace vk

using namespace vk;

VK_API int vk_mlstm_max_dim() { return 256; }

// proj float32 [tokens][N] = q [H dim] | k [H dim] | v [H vdim] | gate [H vdim] | a [H] | b [H];  gate_bias float32 [2H] (a's, then b's);
// state float32 [slots][H dim vdim + H dim + H];  o float32 [tokens][H][vdim + 2] (numerators, n . q, m).  A block a (16 columns, head,
// segment): segments is the step's count, whatever their lengths.  S and n of the state are written here, m by vk_mlstm_gate.
VK_API int vk_mlstm_recurrence(const float* proj, int N, int H, int dim, int vdim, const float* gate_bias, float cap, const int32_t* seg_starts,
                               const int32_t* seg_slots, float* state, float* o, int segments, cudaStream_t stream) {
    if (segments <= 0) return VK_OK;
    if (H <= 0 || dim <= 0 || vdim <= 0 || !(cap > 0.0f) || N < 2 * H * dim + 2 * H * vdim + 2 * H) return VK_BAD_SHAPE;
    if (dim > 256 || H > 65535 || segments > 65535) return VK_TOO_LARGE;
    if ((uintptr_t)proj % 4) return VK_BAD_ALIGNMENT;
    const size_t state_floats = (size_t)H * dim * vdim + (size_t)H * dim + H;
    const float qscale = 1.0f / sqrtf((float)dim);
    const int vec = (N % 4 == 0 && dim % 4 == 0 && vdim % 4 == 0 && (uintptr_t)proj % 16 == 0) ? 1 : 0;    // every piece starts on 16 bytes
    dim3 grid((vdim + 1 + ML_COLS - 1) / ML_COLS, H, segments);
#define VK_MLSTM(D, C)                                                                                                                       \
    do {                                                                                                                                     \
        auto kern = mlstm_recurrence_kernel<D, C>;                                                                                           \
        const size_t smem = 2 * (size_t)ml_stage_floats(C, D) * sizeof(float);                                                               \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                                  \
        if (e != cudaSuccess) return (int)e;                                                                                                 \
        return launch_dependent(kern, grid, dim3(ML_THREADS), smem, stream, proj, N, H, dim, vdim, gate_bias, cap, qscale, seg_starts,       \
                                seg_slots, state, state_floats, o, vec);                                                                     \
    } while (0)
    if (dim <= 32) VK_MLSTM(4, 32);
    if (dim <= 64) VK_MLSTM(8, 32);
    if (dim <= 128) VK_MLSTM(16, 32);
    VK_MLSTM(32, 16);
#undef VK_MLSTM
}

VK_API int vk_mlstm_gate(const float* o, const float* proj, int N, int gate_off, const float* w, float eps, int H, int dim, int vdim, void* out,
                         int tokens, const int32_t* seg_starts, const int32_t* seg_slots, float* state, int segments, int dtype,
                         cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (H <= 0 || dim <= 0 || vdim <= 0 || gate_off < 0 || gate_off + H * vdim > N || segments < 0) return VK_BAD_SHAPE;
    const size_t state_floats = (size_t)H * dim * vdim + (size_t)H * dim + H;
    const dim3 grid(tokens + segments);
    if (dtype == 0)
        return launch_dependent(mlstm_gate_kernel<float>, grid, dim3(256), 0, stream, o, proj, N, gate_off, w, eps, H, dim, vdim, (float*)out, tokens,
                                seg_starts, seg_slots, state, state_floats);
    return launch_dependent(mlstm_gate_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, o, proj, N, gate_off, w, eps, H, dim, vdim,
                            (__nv_bfloat16*)out, tokens, seg_starts, seg_slots, state, state_floats);
}
