// Gated linear attention: a recurrent mixer whose state is, per head, a matrix S [dim][vdim] that decays per key channel.
//
//  a_t = sigmoid(z_t)^(1/tau),  z_t = W_a2 (W_a1 x_t) + b          one decay per head and key channel, in (0, 1)
//  S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t          q scaled by dim^-1/2; S starts at zero
//  out = o / rms(o) per head * w * silu(gate)                      w [vdim], shared by the heads
//
//  gla_prepare      four tokens a block: z from the narrow half W_a1 x (columns of the first product, float32) and the wide half W_a2
//                   (float32, transposed so that neighbouring threads read neighbouring channels), then a = exp(log sigmoid(z) / tau)
//                   to float32 [tokens][H dim].  A channel's sum runs over the rank in one order whatever the batch.
//  gla_recurrence   token after token, one block per (8 or 16 columns, head, segment).  A warp holds 2 or 4 columns; the 16 or 8 lanes
//                   of a column are groups of rows (group g has rows 4 RG j + 4 g .. + 3), so a thread keeps dim / RG values of its
//                   column in registers, reads keys, queries and decays as float4 and a token's sum over the rows ends with four or
//                   three shuffles, which four tokens take together.  Tokens come in
//                   chunks through a ring of two stages in shared memory that cp.async fills a chunk ahead: q, k, a and the block's
//                   columns of v.  A token's step in the chain is multiplications and additions only.  Writes o float32
//                   [tokens][H][vdim] and, after the segment's last token, the state.
//  gla_gate         one block a token, a warp a head: o / rms(o) * w * silu(gate) to the compute dtype.
//  gla_decode       single decoded tokens, one block per (16 columns, head, segment): the decays of the head's channels, one step of
//                   the recurrence and the state's update in one launch (the gate kernel follows).
//
// The state of a slot is float32 [H][dim][vdim].  Everything is float32 with accurate expf and log1pf, and the order of the sums of an
// output does not depend on how the tokens were cut into steps.
#include "common.cuh"

namespace vk {

__device__ __forceinline__ float gla_log_sigmoid(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

constexpr int GLA_THREADS = 128;
constexpr int GLA_PREP_TOKENS = 4;

__device__ __forceinline__ void gla_cp4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void gla_cp16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// proj float32 [tokens][N] with the narrow half at columns a_off .. a_off + rank - 1; a2t float32 [rank][C]; bias float32 [C];
// decay float32 [tokens][C], C = H dim.
__global__ void __launch_bounds__(256) gla_prepare_kernel(const float* __restrict__ proj, int N, int a_off, int rank, const float* __restrict__ a2t,
                                                          const float* __restrict__ bias, float inv_tau, int C, float* __restrict__ decay, int tokens) {
    extern __shared__ float gp_sh[];                    // [GLA_PREP_TOKENS][rank]
    dependency_wait();
    let_dependents_start();
    const int t0 = blockIdx.x * GLA_PREP_TOKENS, cnt = min(GLA_PREP_TOKENS, tokens - t0);
    for (int i = threadIdx.x; i < cnt * rank; i += blockDim.x) gp_sh[i] = proj[(size_t)(t0 + i / rank) * N + a_off + i % rank];
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float z[GLA_PREP_TOKENS];
#pragma unroll
        for (int t = 0; t < GLA_PREP_TOKENS; t++) z[t] = 0.0f;
        for (int j = 0; j < rank; j++) {
            const float w = a2t[(size_t)j * C + c];
#pragma unroll
            for (int t = 0; t < GLA_PREP_TOKENS; t++) z[t] = fmaf(gp_sh[t * rank + j], w, z[t]);
        }
        const float b = bias[c];
#pragma unroll
        for (int t = 0; t < GLA_PREP_TOKENS; t++)
            if (t < cnt) decay[(size_t)(t0 + t) * C + c] = expf(gla_log_sigmoid(z[t] + b) * inv_tau);
    }
}

// Floats of one stage: q [C][RG DPT] | k [C][RG DPT] | a [C][RG DPT] | v [C][columns of a block]
__host__ __device__ constexpr int gla_stage_floats(int C, int DPT, int RG) { return C * (3 * RG * DPT + 4 * (32 / RG)); }

// The sum of a column's rows over the RG lanes that share it: lanes of one column differ by multiples of 32 / RG.
template <int RG>
__device__ __forceinline__ float gla_column_sum(float p) {
#pragma unroll
    for (int off = 32 / RG; off < 32; off <<= 1) p += __shfl_xor_sync(0xffffffffu, p, off);
    return p;
}

// RG lanes share a column (RG = 8: group g has rows 32 j + 4 g .. + 3; RG = 16: rows 64 j + 4 g .. + 3), DPT rows a lane; a warp holds
// 32 / RG columns, a block of four warps 128 / RG.
template <int DPT, int C, int RG>
__global__ void __launch_bounds__(GLA_THREADS) gla_recurrence_kernel(const float* __restrict__ proj, int N, int H, int dim, int vdim,
                                                                     const float* __restrict__ decay, float qscale,
                                                                     const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots,
                                                                     float* __restrict__ state, size_t state_floats, float* __restrict__ o, int vec) {
    constexpr int DP = RG * DPT;                                                // rows of the state as the registers hold them (dim rounded up)
    constexpr int CPW = 32 / RG, COLS = 4 * CPW;                                // columns of a warp and of a block
    constexpr int STAGE = gla_stage_floats(C, DPT, RG);
    extern __shared__ __align__(16) float gla_smem[];
    dependency_wait();
    let_dependents_start();
    const int seg = blockIdx.z, h = blockIdx.y, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int rg = lane / CPW;                                      // rows 4 RG j + 4 rg .. + 3
    const int cl = warp * CPW + lane % CPW;
    const int col0 = blockIdx.x * COLS, col = col0 + cl;
    const int first = seg_starts[seg], end = seg_starts[seg + 1], slot = seg_slots[seg];
    if (first >= end) return;
    float* st = slot >= 0 ? state + (size_t)slot * state_floats : nullptr;
    float* col_st = (!st || col >= vdim) ? nullptr : st + (size_t)h * dim * vdim + col;
    float S[DPT];
#pragma unroll
    for (int j = 0; j < DPT / 4; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int d = 4 * RG * j + 4 * rg + i;
            S[4 * j + i] = (col_st && d < dim) ? col_st[(size_t)d * vdim] : 0.0f;
        }
    const int q_off = h * dim, k_off = H * dim + h * dim, v_off = 2 * H * dim + h * vdim + col0;
    const int v_cnt = min(COLS, vdim - col0);
    // what cp.async never writes: rows beyond dim and columns beyond vdim are zero
    for (int s = 0; s < 2; s++) {
        float* sq = gla_smem + s * STAGE;
        for (int e = tid; e < 3 * C * DP; e += GLA_THREADS)
            if (e % DP >= dim) sq[e] = 0.0f;
        float* sv = sq + 3 * C * DP;
        for (int e = tid; e < C * COLS; e += GLA_THREADS)
            if (col0 + e % COLS >= vdim) sv[e] = 0.0f;
    }
    auto issue = [&](int chunk) {
        float* sq = gla_smem + (chunk & 1) * STAGE;
        float* sk = sq + C * DP;
        float* sa = sk + C * DP;
        float* sv = sa + C * DP;
        const int t0 = first + chunk * C, cnt = min(C, end - t0);
        for (int t = warp; t < cnt; t += GLA_THREADS / 32) {
            const float* row = proj + (size_t)(t0 + t) * N;
            const float* arow = decay + (size_t)(t0 + t) * H * dim + h * dim;
            if (vec) {
                for (int c = 4 * lane; c < dim; c += 128) {
                    gla_cp16(sq + t * DP + c, row + q_off + c);
                    gla_cp16(sk + t * DP + c, row + k_off + c);
                    gla_cp16(sa + t * DP + c, arow + c);
                }
                if (4 * lane < v_cnt) gla_cp16(sv + t * COLS + 4 * lane, row + v_off + 4 * lane);      // COLS is 8 or 16: whole pieces
            } else {
                for (int c = lane; c < dim; c += 32) {
                    gla_cp4(sq + t * DP + c, row + q_off + c);
                    gla_cp4(sk + t * DP + c, row + k_off + c);
                    gla_cp4(sa + t * DP + c, arow + c);
                }
                if (lane < v_cnt) gla_cp4(sv + t * COLS + lane, row + v_off + lane);
            }
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
        const float* sq = gla_smem + (c & 1) * STAGE;
        const float* sk = sq + C * DP;
        const float* sa = sk + C * DP;
        const float* sv = sa + C * DP;
        const int t0 = first + c * C, cnt = min(C, end - t0);
        // a token's step: the column's rows decay, take the key's share of the value, and meet the query; the sum over the rows of the
        // eight lanes that share a column ends with three shuffles, which four tokens take together (the chain is the state's alone)
        auto one = [&](int t) -> float {
            const float vv = sv[t * COLS + cl];
            const float4* k4 = reinterpret_cast<const float4*>(sk + t * DP) + rg;
            const float4* q4 = reinterpret_cast<const float4*>(sq + t * DP) + rg;
            const float4* a4 = reinterpret_cast<const float4*>(sa + t * DP) + rg;
            float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
            for (int j = 0; j < DPT / 4; j++) {
                const float4 kk = k4[RG * j], qq = q4[RG * j], aa = a4[RG * j];
                S[4 * j + 0] = fmaf(kk.x, vv, aa.x * S[4 * j + 0]);
                S[4 * j + 1] = fmaf(kk.y, vv, aa.y * S[4 * j + 1]);
                S[4 * j + 2] = fmaf(kk.z, vv, aa.z * S[4 * j + 2]);
                S[4 * j + 3] = fmaf(kk.w, vv, aa.w * S[4 * j + 3]);
                p0 = fmaf(S[4 * j + 0], qq.x, p0);
                p1 = fmaf(S[4 * j + 1], qq.y, p1);
                p2 = fmaf(S[4 * j + 2], qq.z, p2);
                p3 = fmaf(S[4 * j + 3], qq.w, p3);
            }
            return (p0 + p1) + (p2 + p3);
        };
        int t = 0;
        for (; t + 4 <= cnt; t += 4) {
            float po[4];
#pragma unroll
            for (int u = 0; u < 4; u++) po[u] = one(t + u);
#pragma unroll
            for (int off = CPW; off < 32; off <<= 1) {
#pragma unroll
                for (int u = 0; u < 4; u++) po[u] += __shfl_xor_sync(0xffffffffu, po[u], off);
            }
            if (rg == 0 && col < vdim) {
#pragma unroll
                for (int u = 0; u < 4; u++) o[((size_t)(t0 + t + u) * H + h) * vdim + col] = po[u] * qscale;
            }
        }
        for (; t < cnt; t++) {
            const float po = gla_column_sum<RG>(one(t));
            if (rg == 0 && col < vdim) o[((size_t)(t0 + t) * H + h) * vdim + col] = po * qscale;
        }
        __syncthreads();                                            // the stage is filled again at the top of the next round
    }
    if (!col_st) return;
#pragma unroll
    for (int j = 0; j < DPT / 4; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int d = 4 * RG * j + 4 * rg + i;
            if (d < dim) col_st[(size_t)d * vdim] = S[4 * j + i];
        }
}

// Single decoded tokens: the decays of the head's channels (as gla_prepare sums them), one step, the state's update.  The rows of the
// state are taken in the same groups and summed in the same order as in gla_recurrence, so a token gives the same bits either way.
template <int DPT, int RG>
__global__ void __launch_bounds__(GLA_THREADS) gla_decode_kernel(const float* __restrict__ proj, int N, int H, int dim, int vdim, int a_off, int rank,
                                                                 const float* __restrict__ a2t, const float* __restrict__ bias, float inv_tau,
                                                                 float qscale, const int32_t* __restrict__ seg_starts,
                                                                 const int32_t* __restrict__ seg_slots, float* __restrict__ state, size_t state_floats,
                                                                 float* __restrict__ o) {
    constexpr int DP = RG * DPT;
    constexpr int CPW = 32 / RG, COLS = 4 * CPW;
    __shared__ __align__(16) float sq[DP], sk[DP], sa[DP];
    extern __shared__ float gd_a1[];                                // [rank]
    dependency_wait();
    let_dependents_start();
    const int seg = blockIdx.z, h = blockIdx.y, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5, rg = lane / CPW, cl = warp * CPW + lane % CPW;
    const int col = blockIdx.x * COLS + cl;
    const int t = seg_starts[seg], slot = seg_slots[seg];
    if (t >= seg_starts[seg + 1]) return;
    const float* row = proj + (size_t)t * N;
    for (int j = tid; j < rank; j += GLA_THREADS) gd_a1[j] = row[a_off + j];
    for (int d = tid; d < DP; d += GLA_THREADS) {
        sq[d] = d < dim ? row[h * dim + d] : 0.0f;
        sk[d] = d < dim ? row[H * dim + h * dim + d] : 0.0f;
    }
    __syncthreads();
    const int C = H * dim;
    for (int d = tid; d < DP; d += GLA_THREADS) {
        float a = 0.0f;
        if (d < dim) {
            float z = 0.0f;
            for (int j = 0; j < rank; j++) z = fmaf(gd_a1[j], a2t[(size_t)j * C + h * dim + d], z);
            a = expf(gla_log_sigmoid(z + bias[h * dim + d]) * inv_tau);
        }
        sa[d] = a;
    }
    __syncthreads();
    float* st = slot >= 0 ? state + (size_t)slot * state_floats : nullptr;
    float* col_st = (!st || col >= vdim) ? nullptr : st + (size_t)h * dim * vdim + col;
    const float vv = col < vdim ? row[2 * H * dim + h * vdim + col] : 0.0f;
    const float4* k4 = reinterpret_cast<const float4*>(sk) + rg;
    const float4* q4 = reinterpret_cast<const float4*>(sq) + rg;
    const float4* a4 = reinterpret_cast<const float4*>(sa) + rg;
    float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
    for (int j = 0; j < DPT / 4; j++) {
        const float4 kk = k4[RG * j], qq = q4[RG * j], aa = a4[RG * j];
        const float kv[4] = {kk.x, kk.y, kk.z, kk.w}, av[4] = {aa.x, aa.y, aa.z, aa.w};
        float s[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int d = 4 * RG * j + 4 * rg + i;
            const float old = (col_st && d < dim) ? col_st[(size_t)d * vdim] : 0.0f;
            s[i] = fmaf(kv[i], vv, av[i] * old);
            if (col_st && d < dim) col_st[(size_t)d * vdim] = s[i];
        }
        p0 = fmaf(s[0], qq.x, p0);
        p1 = fmaf(s[1], qq.y, p1);
        p2 = fmaf(s[2], qq.z, p2);
        p3 = fmaf(s[3], qq.w, p3);
    }
    const float po = gla_column_sum<RG>((p0 + p1) + (p2 + p3));
    if (rg == 0 && col < vdim) o[((size_t)t * H + h) * vdim + col] = po * qscale;
}

template <typename T>
__global__ void __launch_bounds__(256) gla_gate_kernel(const float* __restrict__ o, const float* __restrict__ proj, int N, int gate_off,
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
        for (int d = lane; d < vdim; d += 32) {
            const float g = gate[d];
            out[((size_t)t * H + h) * vdim + d] = from_f32<T>(((in[d] * inv) * w[d]) * (g / (1.0f + expf(-g))));
        }
    }
}

}  // namespace vk

using namespace vk;

VK_API int vk_gla_max_dim() { return 256; }

// Sixteen lanes a column (half the rows a lane, half the instructions a token, eight columns a block) where one request's blocks then
// still fit the 148 multiprocessors at once; else eight lanes.  The choice depends on the mixer's sizes alone, never on the batch, and
// the one-launch form for single tokens makes the same one, so that a token's sums meet in one order wherever it is worked out.
static inline bool gla_sixteen_lanes(int H, int dim, int vdim) { return dim > 32 && (long long)((vdim + 7) / 8) * H <= 148; }

// decay float32 [tokens][H dim] <- exp(log sigmoid(a2t^T proj[:, a_off : a_off + rank] + bias) / tau)
VK_API int vk_gla_prepare(const float* proj, int N, int a_off, int rank, const float* a2t, const float* bias, float tau, int channels, float* decay,
                          int tokens, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (rank <= 0 || a_off < 0 || a_off + rank > N || channels <= 0 || !(tau > 0.0f)) return VK_BAD_SHAPE;
    const size_t smem = (size_t)GLA_PREP_TOKENS * rank * sizeof(float);
    if (smem > 48 * 1024) return VK_TOO_LARGE;
    return launch_dependent(gla_prepare_kernel, dim3((tokens + GLA_PREP_TOKENS - 1) / GLA_PREP_TOKENS), dim3(256), smem, stream, proj, N, a_off, rank,
                            a2t, bias, 1.0f / tau, channels, decay, tokens);
}

// proj float32 [tokens][N] = q [H dim] | k [H dim] | v [H vdim] | ...;  decay float32 [tokens][H dim];  state float32 [slots][H dim vdim];
// o float32 [tokens][H][vdim].  A block a (16 columns, head, segment): segments is the step's count, whatever their lengths.
VK_API int vk_gla_recurrence(const float* proj, int N, int H, int dim, int vdim, const float* decay, const int32_t* seg_starts,
                             const int32_t* seg_slots, float* state, float* o, int segments, cudaStream_t stream) {
    if (segments <= 0) return VK_OK;
    if (H <= 0 || dim <= 0 || vdim <= 0 || N < 2 * H * dim + H * vdim) return VK_BAD_SHAPE;
    if (dim > 256 || H > 65535 || segments > 65535) return VK_TOO_LARGE;
    if ((uintptr_t)proj % 4) return VK_BAD_ALIGNMENT;
    const size_t state_floats = (size_t)H * dim * vdim;
    const float qscale = 1.0f / sqrtf((float)dim);
    const int vec = (N % 4 == 0 && dim % 4 == 0 && vdim % 4 == 0 && (uintptr_t)proj % 16 == 0 && (uintptr_t)decay % 16 == 0) ? 1 : 0;
#define VK_GLA(D, C, RG)                                                                                                                     \
    do {                                                                                                                                     \
        auto kern = gla_recurrence_kernel<D, C, RG>;                                                                                         \
        const size_t smem = 2 * (size_t)gla_stage_floats(C, D, RG) * sizeof(float);                                                          \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                                  \
        if (e != cudaSuccess) return (int)e;                                                                                                 \
        const int cols = 128 / RG;                                                                                                           \
        return launch_dependent(kern, dim3((vdim + cols - 1) / cols, H, segments), dim3(GLA_THREADS), smem, stream, proj, N, H, dim, vdim,   \
                                decay, qscale, seg_starts, seg_slots, state, state_floats, o, vec);                                          \
    } while (0)
    if (dim <= 32) VK_GLA(4, 32, 8);
    if (gla_sixteen_lanes(H, dim, vdim)) {
        if (dim <= 64) VK_GLA(4, 32, 16);
        if (dim <= 128) VK_GLA(8, 32, 16);
        VK_GLA(16, 16, 16);
    }
    if (dim <= 64) VK_GLA(8, 32, 8);
    if (dim <= 128) VK_GLA(16, 32, 8);
    VK_GLA(32, 16, 8);
#undef VK_GLA
}

// Every segment is one token: decays, one step and the state's update in one launch.
VK_API int vk_gla_decode(const float* proj, int N, int H, int dim, int vdim, int a_off, int rank, const float* a2t, const float* bias, float tau,
                         const int32_t* seg_starts, const int32_t* seg_slots, float* state, float* o, int segments, cudaStream_t stream) {
    if (segments <= 0) return VK_OK;
    if (H <= 0 || dim <= 0 || vdim <= 0 || N < 2 * H * dim + H * vdim || rank <= 0 || a_off < 0 || a_off + rank > N || !(tau > 0.0f)) return VK_BAD_SHAPE;
    if (dim > 256 || H > 65535 || segments > 65535) return VK_TOO_LARGE;
    const size_t smem = (size_t)rank * sizeof(float);
    if (smem > 32 * 1024) return VK_TOO_LARGE;
    const size_t state_floats = (size_t)H * dim * vdim;
    const float qscale = 1.0f / sqrtf((float)dim);
#define VK_GLAD(D, RG)                                                                                                                        \
    return launch_dependent(gla_decode_kernel<D, RG>, dim3((vdim + 128 / RG - 1) / (128 / RG), H, segments), dim3(GLA_THREADS), smem, stream, proj, N, H, \
                            dim, vdim, a_off, rank, a2t, bias, 1.0f / tau, qscale, seg_starts, seg_slots, state, state_floats, o)
    if (dim <= 32) VK_GLAD(4, 8);
    if (gla_sixteen_lanes(H, dim, vdim)) {
        if (dim <= 64) VK_GLAD(4, 16);
        if (dim <= 128) VK_GLAD(8, 16);
        VK_GLAD(16, 16);
    }
    if (dim <= 64) VK_GLAD(8, 8);
    if (dim <= 128) VK_GLAD(16, 8);
    VK_GLAD(32, 8);
#undef VK_GLAD
}

// out [tokens][H vdim] in dtype = o / rms(o) per head * w [vdim] * silu(proj[:, gate_off + ...])
VK_API int vk_gla_gate(const float* o, const float* proj, int N, int gate_off, const float* w, float eps, int H, int vdim, void* out, int tokens,
                       int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (H <= 0 || vdim <= 0 || gate_off < 0 || gate_off + H * vdim > N) return VK_BAD_SHAPE;
    if (dtype == 0)
        return launch_dependent(gla_gate_kernel<float>, dim3(tokens), dim3(256), 0, stream, o, proj, N, gate_off, w, eps, H, vdim, (float*)out);
    return launch_dependent(gla_gate_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, o, proj, N, gate_off, w, eps, H, vdim,
                            (__nv_bfloat16*)out);
}
