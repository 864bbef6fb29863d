// A routed feed-forward: every token uses `top` of E small gated feed-forward layers, weighted by a softmax over the chosen logits.
//
//  experts_route     one block a token: logits z = W_r x + b in float32 (a warp a logit), the `top` largest (of equal logits the lower
//                    index), weights = softmax over the chosen logits alone.  Writes ids [tokens][top] and weights [tokens][top].
//  experts_route_table  ids[token][k] = table[token id][k], every weight 1 / top: the experts of a token are a function of its id.
//  experts_gate_up   act[token, k] = f(W_gate,e x) * (W_up,e x) for the token's k-th expert e; a warp an output column, the token's row
//                    in shared memory.  f is one of the epilogues' activations.
//  experts_down      y[token] += sum_k weight_k W_down,e_k act[token, k], the experts of a token summed in the order of its list, so
//                    that the sum does not depend on what else is in the batch.
//
// For a prompt's portion in bfloat16 the experts' products run on the tensor cores as products of row groups (linear_tcgen05.cu):
//  experts_sort      one block: counts the copies a group (an expert) gets, gives every group whole tiles of 128 rows one after another,
//                    and writes for each (token, k) its row, for each row its token (-1: a fill row), for each tile its group
//                    (-1: unused).  Which copy of a group gets which of its rows is left to the order of arrival: a row's product
//                    does not depend on where in a tile it stands.
//  experts_gather    a block a row: the token's input row is copied to its row of the grouped matrix.
//  experts_combine   a block a token: y[token] += sum_k weight_k out[row of (token, k)], in the order of the token's list.
//
// Nothing here comes to the host: which experts run is read by the kernels from the ids on the device, so a captured graph
// replays the part for any batch.  Products accumulate in float32 (fmaf); storage is float32 or bfloat16.
#include "common.cuh"

namespace vk {

template <typename T>
__global__ void __launch_bounds__(128) experts_route_kernel(const T* __restrict__ x, int width, const float* __restrict__ wr,
                                                            const float* __restrict__ br, int E, int top, int32_t* __restrict__ ids,
                                                            float* __restrict__ wts) {
    extern __shared__ float z[];                        // [E]
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const T* row = x + (size_t)t * width;
    for (int e = warp; e < E; e += nwarps) {
        const float* w = wr + (size_t)e * width;
        float acc = 0.0f;
        for (int i = lane; i < width; i += 32) acc = fmaf(to_f32<T>(row[i]), w[i], acc);
        acc = warp_sum(acc);
        if (lane == 0) z[e] = acc + (br ? br[e] : 0.0f);
    }
    __syncthreads();
    if (warp != 0) return;
    // the warp picks the largest logit `top` times; every lane knows each pick, lane k keeps the k-th weight
    __shared__ int picked[32];
    float zmax = 0.0f, sum = 0.0f, mine = 0.0f;
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < arg)) {
                bool taken = false;
                for (int j = 0; j < k; j++) taken |= picked[j] == e;
                if (!taken) { best = v; arg = e; }
            }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg == 0x7fffffff) arg = 0;                 // logits that are not numbers: stay inside the tables
        if (k == 0) zmax = best;
        const float p = expf(best - zmax);
        sum += p;
        if (lane == k) mine = p;
        if (lane == 0) picked[k] = arg;
        __syncwarp();
    }
    if (lane < top) {
        ids[(size_t)t * top + lane] = picked[lane];
        wts[(size_t)t * top + lane] = mine / sum;
    }
}

__global__ void __launch_bounds__(256) experts_route_table_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ table, int vocab,
                                                                  int table_top, int E, int top, int32_t* __restrict__ ids, float* __restrict__ wts, int n) {
    dependency_wait();
    let_dependents_start();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int t = i / top, k = i - t * top;
    int id = tokens[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    int e = table[(size_t)id * table_top + k];
    ids[i] = e < 0 ? 0 : (e >= E ? E - 1 : e);         // a table that names no expert of the layer: stay inside the weights
    wts[i] = 1.0f / (float)top;
}

// grid (pairs, column groups); a warp a column
template <typename T>
__global__ void __launch_bounds__(256) experts_gate_up_kernel(const T* __restrict__ x, int width, const T* __restrict__ wgu, int ff, int top,
                                                              const int32_t* __restrict__ ids, int act, float limit, float alpha,
                                                              T* __restrict__ out) {
    extern __shared__ float xs[];                       // [width]
    dependency_wait();
    let_dependents_start();
    const int p = blockIdx.x, t = p / top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < width; i += blockDim.x) xs[i] = to_f32<T>(x[(size_t)t * width + i]);
    __syncthreads();
    const int e = ids[p];
    const T* wg = wgu + (size_t)e * 2 * ff * width;
    const T* wu = wg + (size_t)ff * width;
    for (int c = blockIdx.y * nwarps + warp; c < ff; c += gridDim.y * nwarps) {
        const T* g = wg + (size_t)c * width;
        const T* u = wu + (size_t)c * width;
        float ag = 0.0f, au = 0.0f;
        for (int i = lane; i < width; i += 32) {
            ag = fmaf(xs[i], to_f32<T>(g[i]), ag);
            au = fmaf(xs[i], to_f32<T>(u[i]), au);
        }
        ag = warp_sum(ag);
        au = warp_sum(au);
        if (lane == 0) {
            float r;
            if (act == 4) {                             // the clamped form: min(g, L) sigmoid(alpha min(g, L)) (clamp(u, -L, L) + 1)
                const float g = fminf(ag, limit), u = fminf(fmaxf(au, -limit), limit);
                r = (g / (1.0f + expf(-alpha * g))) * (u + 1.0f);
            } else {
                r = activate_rt(act, ag) * au;
            }
            out[(size_t)p * ff + c] = from_f32<T>(r);
        }
    }
}

// grid (tokens, column groups); a warp a column of y
template <typename T>
__global__ void __launch_bounds__(256) experts_down_kernel(const T* __restrict__ act, int ff, const T* __restrict__ wd, int width, int top,
                                                           const int32_t* __restrict__ ids, const float* __restrict__ wts, float* __restrict__ y) {
    extern __shared__ float as[];                       // [top][ff]
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) as[i] = to_f32<T>(act[(size_t)t * top * ff + i]);
    __syncthreads();
    for (int c = blockIdx.y * nwarps + warp; c < width; c += gridDim.y * nwarps) {
        float total = 0.0f;
        for (int k = 0; k < top; k++) {
            const int e = ids[(size_t)t * top + k];
            const T* w = wd + ((size_t)e * width + c) * ff;
            const float* a = as + (size_t)k * ff;
            float acc = 0.0f;
            for (int i = lane; i < ff; i += 32) acc = fmaf(a[i], to_f32<T>(w[i]), acc);
            total = fmaf(wts[(size_t)t * top + k], warp_sum(acc), total);
        }
        if (lane == 0) y[(size_t)t * width + c] += total;
    }
}

constexpr int EXPERT_TILE = 128;                        // rows of a tile of the grouped products

__global__ void __launch_bounds__(1024) experts_sort_kernel(const int32_t* __restrict__ ids, int n, int E, int rows_max, int32_t* __restrict__ pos,
                                                            int32_t* __restrict__ row_token, int32_t* __restrict__ tile_group, int top) {
    extern __shared__ int sort_sh[];                    // count [E] | start [E]
    int* count = sort_sh;
    int* start = sort_sh + E;
    dependency_wait();
    let_dependents_start();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    for (int i = threadIdx.x; i < rows_max; i += blockDim.x) row_token[i] = -1;
    for (int i = threadIdx.x; i < rows_max / EXPERT_TILE; i += blockDim.x) tile_group[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; e++) {
            start[e] = at;
            at += (count[e] + EXPERT_TILE - 1) / EXPERT_TILE * EXPERT_TILE;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        for (int r = start[e]; r < start[e] + count[e] && r < rows_max; r += EXPERT_TILE) tile_group[r / EXPERT_TILE] = e;
        count[e] = 0;                                   // from here on: the rows of the group that are taken
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = ids[i];
        int r = -1;
        if (e >= 0 && e < E) {
            r = start[e] + atomicAdd(&count[e], 1);
            if (r < rows_max) row_token[r] = i / top; else r = -1;
        }
        pos[i] = r;
    }
}

template <typename T>
__global__ void __launch_bounds__(128) experts_gather_kernel(const T* __restrict__ x, int width, const int32_t* __restrict__ row_token,
                                                             T* __restrict__ xs) {
    dependency_wait();
    let_dependents_start();
    const int t = row_token[blockIdx.x];
    if (t < 0) return;
    const T* src = x + (size_t)t * width;
    T* dst = xs + (size_t)blockIdx.x * width;
    constexpr int V = Vec16<T>::N;
    if (width % V == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)xs % 16 == 0)) {
        for (int i = threadIdx.x; i < width / V; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
    }
}

__global__ void __launch_bounds__(256) experts_combine_kernel(const float* __restrict__ o, int width, int top, const int32_t* __restrict__ pos,
                                                              const float* __restrict__ wts, float* __restrict__ y) {
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float total = 0.0f;
        for (int k = 0; k < top; k++) {
            const int r = pos[(size_t)t * top + k];
            if (r >= 0) total = fmaf(wts[(size_t)t * top + k], o[(size_t)r * width + c], total);
        }
        y[(size_t)t * width + c] += total;
    }
}

}  // namespace vk

using namespace vk;

// Rows that the grouped matrix needs for `tokens` tokens at most: every copy, and every group filled up to a whole tile.
VK_API int vk_experts_grouped_rows(int tokens, int top, int E) {
    const long long rows = ((long long)tokens * top + (long long)E * (EXPERT_TILE - 1) + EXPERT_TILE - 1) / EXPERT_TILE * EXPERT_TILE;
    return rows > 0x7fffffffLL ? -1 : (int)rows;
}

// ids int32 [tokens][top] -> pos int32 [tokens][top], row_token int32 [rows_max], tile_group int32 [rows_max / 128];
// rows_max = vk_experts_grouped_rows(tokens, top, E).
VK_API int vk_experts_sort(const int32_t* ids, int tokens, int top, int E, int rows_max, int32_t* pos, int32_t* row_token, int32_t* tile_group,
                           cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (top <= 0 || E <= 0 || rows_max < vk_experts_grouped_rows(tokens, top, E) || rows_max % EXPERT_TILE) return VK_BAD_SHAPE;
    const size_t smem = 2 * (size_t)E * sizeof(int);
    if (smem > 48 * 1024) return VK_TOO_LARGE;
    return launch_dependent(experts_sort_kernel, dim3(1), dim3(1024), smem, stream, ids, tokens * top, E, rows_max, pos, row_token, tile_group, top);
}

// xs [rows][width] in dtype <- x [tokens][width] by row_token.
VK_API int vk_experts_gather(const void* x, int width, const int32_t* row_token, void* xs, int rows, int dtype, cudaStream_t stream) {
    if (rows <= 0) return VK_OK;
    if (width <= 0) return VK_BAD_SHAPE;
    if (dtype == 0) return launch_dependent(experts_gather_kernel<float>, dim3(rows), dim3(128), 0, stream, (const float*)x, width, row_token, (float*)xs);
    return launch_dependent(experts_gather_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, stream, (const __nv_bfloat16*)x, width, row_token,
                            (__nv_bfloat16*)xs);
}

// y float32 [tokens][width] += sum_k wts[t][k] o[pos[t][k]]; o float32 [rows][width].
VK_API int vk_experts_combine(const float* o, int width, int top, const int32_t* pos, const float* wts, float* y, int tokens, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (width <= 0 || top <= 0) return VK_BAD_SHAPE;
    return launch_dependent(experts_combine_kernel, dim3(tokens), dim3(256), 0, stream, o, width, top, pos, wts, y);
}

// x [tokens][width] in dtype; wr float32 [E][width], br float32 [E] or null; ids int32 [tokens][top], wts float32 [tokens][top].
VK_API int vk_experts_route(const void* x, int width, const float* wr, const float* br, int E, int top, int32_t* ids, float* wts, int tokens,
                            int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (width <= 0 || E <= 0 || top <= 0 || top > E || top > 32) return VK_BAD_SHAPE;
    const size_t smem = (size_t)E * sizeof(float);
    if (smem > 48 * 1024) return VK_TOO_LARGE;
    if (dtype == 0) return launch_dependent(experts_route_kernel<float>, dim3(tokens), dim3(128), smem, stream, (const float*)x, width, wr, br, E, top, ids, wts);
    return launch_dependent(experts_route_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), smem, stream, (const __nv_bfloat16*)x, width, wr, br, E, top,
                            ids, wts);
}

// tokens int32 [n_tokens] (token ids); table int32 [vocab][table_top], table_top >= top; ids int32 [n_tokens][top], wts float32 [n_tokens][top].
VK_API int vk_experts_route_table(const int32_t* tokens, const int32_t* table, int vocab, int table_top, int E, int top, int32_t* ids, float* wts,
                                  int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return VK_OK;
    if (vocab <= 0 || E <= 0 || top <= 0 || top > table_top) return VK_BAD_SHAPE;
    const int n = n_tokens * top;
    return launch_dependent(experts_route_table_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, tokens, table, vocab, table_top, E, top, ids, wts, n);
}

// wgu [E][2 ff][width] (an expert's gate rows, then its up rows) in dtype; out [tokens * top][ff] in dtype.  act: 0 none, 1 gelu (erf),
// 2 gelu (tanh), 3 silu, 4 the clamped form min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u, -limit, limit) + 1).
VK_API int vk_experts_gate_up(const void* x, int width, const void* wgu, int ff, int top, const int32_t* ids, int act, float limit, float alpha,
                              void* out, int tokens, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (width <= 0 || ff <= 0 || top <= 0 || act < 0 || act > 4 || (act == 4 && !(limit > 0.0f))) return VK_BAD_SHAPE;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 48 * 1024) return VK_TOO_LARGE;
    int gy = (ff + 7) / 8;
    if (gy > 64) gy = 64;
    dim3 grid(tokens * top, gy);
    if (dtype == 0)
        return launch_dependent(experts_gate_up_kernel<float>, grid, dim3(256), smem, stream, (const float*)x, width, (const float*)wgu, ff, top, ids, act,
                                limit, alpha, (float*)out);
    return launch_dependent(experts_gate_up_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)x, width,
                            (const __nv_bfloat16*)wgu, ff, top, ids, act, limit, alpha, (__nv_bfloat16*)out);
}

// act [tokens * top][ff] and wd [E][width][ff] in dtype; y float32 [tokens][width] is added to.
VK_API int vk_experts_down(const void* act, int ff, const void* wd, int width, int top, const int32_t* ids, const float* wts, float* y, int tokens,
                           int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (width <= 0 || ff <= 0 || top <= 0) return VK_BAD_SHAPE;
    const size_t smem = (size_t)top * ff * sizeof(float);
    if (smem > 48 * 1024) return VK_TOO_LARGE;
    int gy = (width + 7) / 8;
    if (gy > 64) gy = 64;
    dim3 grid(tokens, gy);
    if (dtype == 0)
        return launch_dependent(experts_down_kernel<float>, grid, dim3(256), smem, stream, (const float*)act, ff, (const float*)wd, width, top, ids, wts, y);
    return launch_dependent(experts_down_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)act, ff, (const __nv_bfloat16*)wd,
                            width, top, ids, wts, y);
}
