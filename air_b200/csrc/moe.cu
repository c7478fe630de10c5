// Routing of a mixture of experts, on the device from start to end (nothing is read on the host, so a step can be
// captured in a CUDA graph).
//
// moe_route_kernel: from the router's logits z [T, ld] (float32; the first n columns, and at column n, where the
//   layer has one, the logit of a gate for a shared expert) to each token's `top` experts with the largest scores.
//   score 0 is sigmoid(z), score 1 the softmax over the n logits; the weights are the chosen scores as they are, or
//   (renormalize) divided by their sum (+ norm_eps), and then times route_scale.  Equal scores: the lower index wins.
//   With groups > 1 experts g * (n / groups) .. (g + 1) * (n / groups) - 1 make group g; a group's mark is its best score
//   plus its second best (its only score where a group is one expert), and only the experts of the `keep` groups with the
//   largest marks (of equal marks the lower group) can be chosen.  One warp per token.
//   With a bias (float32 [n]) the experts are chosen by score + bias, while the weights stay the scores themselves.
//   Writes expert [T, top] int32, weight [T, top] float32 and gate [T] = sigmoid(z[n]).
//
// moe_identity_kernel: experts with an index of n_real or more have no matrices: their output is their input.  For
//   every (token, choice) pair of such an expert: y[choice][token][:] = weight * x[token][:] (y float32 planes).
//
// moe_sort_kernel: orders the T * top (token, choice) pairs by expert.  Writes start [n + 1] (the slots of expert e are
//   start[e] .. start[e + 1]), pair_of_slot [T * top] (pair = token * top + choice), and the list of row tiles of
//   `tile_rows` slots that the grouped matrix product walks: tiles [2 * i] = expert, [2 * i + 1] = first slot, and
//   their number.  Pairs of an expert outside 0 .. n - 1 get no slot; the slots behind the last one hold -1.  One
//   block.  Inside an expert the order of the slots is whatever the atomic counters give; a row of
//   a product does not depend on its neighbours, so the result does not depend on it.
#include "common.cuh"

namespace air {

constexpr int MOE_MAX_PER_LANE = 16;      // up to 512 experts

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ z, int ld, int T, int n, int top, int score, int renormalize,
                 int has_gate, int* __restrict__ expert, float* __restrict__ weight, float* __restrict__ gate,
                 int groups, int keep, float route_scale, float norm_eps, const float* __restrict__ bias) {
    __shared__ float held[4][32 * MOE_MAX_PER_LANE], marks[4][32 * MOE_MAX_PER_LANE];
    pdl_enter(TR_MOE_ROUTE);
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const float* row = z + (size_t)t * ld;
    float s[MOE_MAX_PER_LANE];
    float zmax = -INFINITY;
#pragma unroll
    for (int c = 0; c < MOE_MAX_PER_LANE; ++c) {
        const int e = lane + 32 * c;
        s[c] = e < n ? row[e] : -INFINITY;
        zmax = fmaxf(zmax, s[c]);
    }
    if (score == 1) {
        zmax = warp_max(zmax);
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < MOE_MAX_PER_LANE; ++c) {
            s[c] = lane + 32 * c < n ? expf(s[c] - zmax) : 0.f;
            sum += s[c];
        }
        sum = warp_sum(sum);
#pragma unroll
        for (int c = 0; c < MOE_MAX_PER_LANE; ++c) s[c] /= sum;
    } else {
#pragma unroll
        for (int c = 0; c < MOE_MAX_PER_LANE; ++c) s[c] = 1.f / (1.f + expf(-s[c]));
    }
    // ch: what the experts are chosen by (the score, plus the bias where there is one); s stays the weight
    constexpr float NEVER = -3.0e38f;
    float ch[MOE_MAX_PER_LANE];
#pragma unroll
    for (int c = 0; c < MOE_MAX_PER_LANE; ++c) {
        const int e = lane + 32 * c;
        if (e >= n || !(s[c] == s[c])) {      // outside, or not a number: never preferred
            s[c] = 0.f;
            ch[c] = NEVER;
        } else {
            ch[c] = bias ? s[c] + bias[e] : s[c];
        }
    }
    if (groups > 1) {
        float* my = held[threadIdx.x >> 5];
        float* mk = marks[threadIdx.x >> 5];
        const int size = n / groups;
#pragma unroll
        for (int c = 0; c < MOE_MAX_PER_LANE; ++c)
            if (lane + 32 * c < n) my[lane + 32 * c] = ch[c] == NEVER ? -1.f : ch[c];
        __syncwarp();
        for (int g = lane; g < groups; g += 32) {
            float a = -1.f, b = -1.f;      // the group's two largest scores
            for (int i = 0; i < size; ++i) {
                const float v = my[g * size + i];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            mk[g] = size > 1 ? a + b : a;
        }
        __syncwarp();
        // a group takes part if fewer than `keep` groups come before it (a larger mark, or an equal one and a lower
        // index); the scores in `my` have been read, so the flags go there
        for (int g = lane; g < groups; g += 32) {
            int before = 0;
            for (int o = 0; o < groups; ++o) before += (mk[o] > mk[g] || (mk[o] == mk[g] && o < g)) ? 1 : 0;
            my[g] = before < keep ? 1.f : 0.f;
        }
        __syncwarp();
#pragma unroll
        for (int c = 0; c < MOE_MAX_PER_LANE; ++c) {
            const int e = lane + 32 * c;
            if (e < n && my[e / size] == 0.f) ch[c] = NEVER;
        }
    }
    float total = 0.f;
    float mine = 0.f;      // lane j keeps the weight of choice j
    int mine_e = 0;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int best_e = n;
#pragma unroll
        for (int c = 0; c < MOE_MAX_PER_LANE; ++c) {
            const int e = lane + 32 * c;
            if (e < n && ch[c] > best) { best = ch[c]; best_e = e; }      // ascending e: the first of equals stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        float own = 0.f;      // the chosen expert's score, held by the lane that has it
#pragma unroll
        for (int c = 0; c < MOE_MAX_PER_LANE; ++c)
            if (lane + 32 * c == best_e) {
                own = s[c];
                ch[c] = -INFINITY;      // taken
            }
        const float wj = fmaxf(__shfl_sync(0xffffffffu, own, best_e & 31), 0.f);
        total += wj;
        if (lane == (j & 31)) {
            if (j >= 32) {      // (more than 32 choices: written as they come)
                expert[(size_t)t * top + j] = best_e;
                weight[(size_t)t * top + j] = wj * route_scale;
            } else {
                mine = wj;
                mine_e = best_e;
            }
        }
    }
    if (lane < top && lane < 32) {
        expert[(size_t)t * top + lane] = mine_e;
        weight[(size_t)t * top + lane] = (renormalize ? mine / (total + norm_eps) : mine) * route_scale;
    }
    if (gate && lane == 0) gate[t] = has_gate ? 1.f / (1.f + expf(-row[n])) : 1.f;
}

__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ expert, int pairs, int n, int tile_rows, int* __restrict__ start,
                int* __restrict__ pair_of_slot, int* __restrict__ tiles, int* __restrict__ num_tiles) {
    extern __shared__ int counts[];      // [n] counts, then [n] fill
    int* fill = counts + n;
    pdl_enter(TR_MOE_SORT);
    for (int e = threadIdx.x; e < 2 * n; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = expert[p];
        if (e >= 0 && e < n) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, nt = 0;
        for (int e = 0; e < n; ++e) {
            const int c = counts[e];
            start[e] = at;
            fill[e] = at;
            for (int r = 0; r < c; r += tile_rows) {
                tiles[2 * nt] = e;
                tiles[2 * nt + 1] = at + r;
                ++nt;
            }
            at += c;
        }
        start[n] = at;
        *num_tiles = nt;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = expert[p];
        if (e >= 0 && e < n) pair_of_slot[atomicAdd(&fill[e], 1)] = p;
    }
    for (int p = start[n] + threadIdx.x; p < pairs; p += blockDim.x) pair_of_slot[p] = -1;      // slots that no pair has
}

// y [top][T][E] float32; x [T, E]; expert, weight [T * top].  One block per pair.
template <typename T>
__global__ void __launch_bounds__(256)
moe_identity_kernel(const T* __restrict__ x, const int* __restrict__ expert, const float* __restrict__ weight,
                    int n_real, int top, size_t plane, float* __restrict__ y, int E) {
    pdl_enter(TR_MOE_SORT);
    const int p = blockIdx.x;
    if (expert[p] < n_real) return;
    const float m = weight[p];
    const T* src = x + (size_t)(p / top) * E;
    float* dst = y + (size_t)(p % top) * plane + (size_t)(p / top) * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x) dst[i] = to_float(src[i]) * m;
}

// rows_by_index_kernel: out[s, :] = x[index[s] / div, :] * scale[index[s]] (scale may be absent), in out's type: a
// token's row once per choice, in the experts' order, with the choice's weight on it.
template <typename T>
__global__ void __launch_bounds__(256)
rows_by_index_kernel(const T* __restrict__ x, const int* __restrict__ index, int div, const float* __restrict__ scale,
                     T* __restrict__ out, int E) {
    pdl_enter(TR_MOE_SORT);
    const int s = blockIdx.x, p = index[s];
    if (p < 0) {      // a slot that no pair has
        for (int i = threadIdx.x; i < E; i += blockDim.x) out[(size_t)s * E + i] = from_float<T>(0.f);
        return;
    }
    const float m = scale ? scale[p] : 1.f;
    const T* src = x + (size_t)(p / div) * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x) out[(size_t)s * E + i] = from_float<T>(to_float(src[i]) * m);
}

// planes_by_index_kernel: out[index[s] % div][index[s] / div][:] = rows[s][:] * scale[index[s]] (out float32; scale
// may be absent): the experts' outputs back to one plane per choice, row = token.
template <typename T>
__global__ void __launch_bounds__(256)
planes_by_index_kernel(const T* __restrict__ rows, const int* __restrict__ index, int div, size_t plane,
                       const float* __restrict__ scale, float* __restrict__ out, int E) {
    pdl_enter(TR_MOE_SORT);
    const int s = blockIdx.x, p = index[s];
    if (p < 0) return;
    const float m = scale ? scale[p] : 1.f;
    float* dst = out + (size_t)(p % div) * plane + (size_t)(p / div) * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x) dst[i] = to_float(rows[(size_t)s * E + i]) * m;
}

}  // namespace air

AIR_API int air_rows_by_index(const void* x, int dtype, const int* index, int div, const float* scale, void* out,
                              int rows, int E, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (div <= 0) return AIR_ERR_BAD_ARGUMENT;
    AIR_DISPATCH(dtype, TT, return air::launch(air::rows_by_index_kernel<TT>, rows, 256, 0, stream, (const TT*)x, index,
                                               div, scale, (TT*)out, E));
    return 0;
}

AIR_API int air_planes_by_index(const void* rows, int dtype, const int* index, int div, long long plane,
                                const float* scale, float* out, int n, int E, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (div <= 0) return AIR_ERR_BAD_ARGUMENT;
    AIR_DISPATCH(dtype, TT, return air::launch(air::planes_by_index_kernel<TT>, n, 256, 0, stream, (const TT*)rows, index,
                                               div, (size_t)plane, scale, out, E));
    return 0;
}

AIR_API int air_moe_route(const float* z, int ld, int T, int n, int top, int score, int renormalize, int has_gate,
                          int* expert, float* weight, float* gate, int groups, int keep, float route_scale,
                          float norm_eps, const float* bias, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n <= 0 || n > 32 * air::MOE_MAX_PER_LANE || top <= 0 || top > n || top > 32 || ld < n + (has_gate ? 1 : 0) ||
        score < 0 || score > 1)
        return AIR_ERR_BAD_ARGUMENT;
    if (groups > 1 && (n % groups || keep <= 0 || keep > groups || top > keep * (n / groups))) return AIR_ERR_BAD_ARGUMENT;
    return air::launch(air::moe_route_kernel, (T + 3) / 4, 128, 0, stream, z, ld, T, n, top, score, renormalize,
                       has_gate, expert, weight, gate, groups, keep, route_scale, norm_eps, bias);
}

AIR_API int air_moe_identity(const void* x, int dtype, const int* expert, const float* weight, int n_real, int top,
                             int T, int E, float* y, cudaStream_t stream) {
    if (T <= 0 || top <= 0) return 0;
    AIR_DISPATCH(dtype, TT, return air::launch(air::moe_identity_kernel<TT>, T * top, 256, 0, stream, (const TT*)x,
                                               expert, weight, n_real, top, (size_t)T * E, y, E));
    return 0;
}

AIR_API int air_moe_sort(const int* expert, int pairs, int n, int tile_rows, int* start, int* pair_of_slot, int* tiles,
                         int* num_tiles, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (n <= 0 || n > 4096 || tile_rows <= 0) return AIR_ERR_BAD_ARGUMENT;
    return air::launch(air::moe_sort_kernel, 1, 1024, sizeof(int) * 2 * (size_t)n, stream, expert, pairs, n, tile_rows,
                       start, pair_of_slot, tiles, num_tiles);
}

AIR_API int air_trace_set_moe(unsigned long long* buffer) { return air::set_trace_here(buffer); }
