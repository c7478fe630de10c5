// Row-wise operations of layers that carry a norm on BOTH sides of every sub-layer, and two small activations.
//
//   normed_add_norm_kernel  d = the sub-layer's output (float32 [T, E], or the partial sums [parts, T, E] of a split
//                           product or the planes of a token's experts, added in order);
//                           x = h + d / sqrt(mean(d^2) + eps_b) * wb      (the norm behind the sub-layer, then the sum)
//                           out = x / sqrt(mean(x^2) + eps) * w            (the norm ahead of the next sub-layer)
//                           x is written back into the stream h when no rows are named; with `rows` the kernel reads
//                           row rows[r] of h and d and leaves h alone.  Without w it only completes the stream.
//                           Everything is 32-bit; out is written in its own type.  A block per row, the row in shared
//                           memory between the passes.
//   relu2_kernel            out = max(x, 0)^2, element by element (float32 or bfloat16 in, out's type out)
//   sigmoid_gate_kernel     x[t, c] *= 1 / (1 + exp(-g[t, c])) in place; g float32 with a row stride of its own (a band of
//                           columns of a wider product); rows whose token_seq is negative are padding
#include "common.cuh"

namespace air {

// VEC: four columns per access (E and the parts' stride multiples of 4, all pointers on 16-byte boundaries).
template <typename TO, bool VEC>
__global__ void normed_add_norm_kernel(float* __restrict__ h, const float* __restrict__ a, int a_parts,
                                       size_t part_stride, const float* __restrict__ wb, float eps_b,
                                       const float* __restrict__ w, TO* __restrict__ out,
                                       const int* __restrict__ rows, int E, float eps) {
    __shared__ float scratch[32];
    extern __shared__ __align__(16) float xrow[];
    pdl_enter(TR_SANDWICH_NORM);
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * E;
    const bool keep = !rows;
    float ss = 0.f;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
            float t[4], u[4];
            load4(a + src + i, t);
#pragma unroll 4
            for (int p = 1; p < a_parts; ++p) {                                   // (loads ahead, sums in order)
                load4(a + p * part_stride + src + i, u);
#pragma unroll
                for (int j = 0; j < 4; ++j) t[j] += u[j];
            }
            store4(xrow + i, t);
#pragma unroll
            for (int j = 0; j < 4; ++j) ss = fmaf(t[j], t[j], ss);
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            float t = a[src + i];
#pragma unroll 4
            for (int p = 1; p < a_parts; ++p) t += a[p * part_stride + src + i];
            xrow[i] = t;
            ss = fmaf(t, t, ss);
        }
    }
    const float rd = 1.f / sqrtf(block_sum(ss, scratch) / (float)E + eps_b);
    ss = 0.f;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
            float x[4], t[4], wv[4];
            load4(h + src + i, x);
            load4(xrow + i, t);
            load4(wb + i, wv);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                x[j] += t[j] * rd * wv[j];
                ss = fmaf(x[j], x[j], ss);
            }
            store4(xrow + i, x);
            if (keep) store4(h + src + i, x);
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            const float x = h[src + i] + xrow[i] * rd * wb[i];
            xrow[i] = x;
            ss = fmaf(x, x, ss);
            if (keep) h[src + i] = x;
        }
    }
    if (!w) return;
    const float scale = 1.f / sqrtf(block_sum(ss, scratch) / (float)E + eps);
    if (VEC) {
        for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
            float x[4], wv[4];
            load4(xrow + i, x);
            load4(w + i, wv);
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] = x[j] * scale * wv[j];
            store4(out + (size_t)r * E + i, x);
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x)
            out[(size_t)r * E + i] = from_float<TO>(xrow[i] * scale * w[i]);
    }
}

template <typename TI, typename TO>
__global__ void relu2_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t total, int vec) {
    pdl_enter(TR_RELU2);
    const size_t step = (size_t)gridDim.x * blockDim.x;
    if (vec) {
        for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total; i += step * 4) {
            float x[4];
            load4(in + i, x);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float r = fmaxf(x[j], 0.f);
                x[j] = r * r;
            }
            store4(out + i, x);
        }
        return;
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const float r = fmaxf(to_float(in[i]), 0.f);
        out[i] = from_float<TO>(r * r);
    }
}

template <typename TX>
__global__ void sigmoid_gate_kernel(TX* __restrict__ x, const float* __restrict__ g, int ldg,
                                    const int* __restrict__ token_seq, int C, size_t total, int vec) {
    pdl_enter(TR_HEAD_GATE);
    const size_t step = (size_t)gridDim.x * blockDim.x;
    if (vec) {
        for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total; i += step * 4) {
            const size_t t = i / C;
            if (token_seq[t] < 0) continue;
            float v[4], gv[4];
            load4(x + i, v);
            load4(g + t * ldg + i % C, gv);
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = v[j] / (1.f + expf(-gv[j]));
            store4(x + i, v);
        }
        return;
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const size_t t = i / C;
        if (token_seq[t] < 0) continue;
        x[i] = from_float<TX>(to_float(x[i]) / (1.f + expf(-g[t * ldg + i % C])));
    }
}

}  // namespace air

AIR_API int air_normed_add_norm(float* h, const float* a, int a_parts, long long part_stride, const float* wb,
                                float eps_b, const float* w, void* out, int out_dtype, const int* rows, int R, int E,
                                float eps, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (!a || !wb || a_parts < 1) return AIR_ERR_BAD_ARGUMENT;
    // few rows: a block as wide as half a row, so that a row's loads are all under way at once
    int threads = E >= 1024 ? 256 : 128;
    if (R <= 256) threads = E / 2 >= 1024 ? 1024 : (E / 2 > threads ? (E / 2 + 31) / 32 * 32 : threads);
    const size_t smem = sizeof(float) * (size_t)E;
    if (smem > 200 * 1024) return AIR_ERR_BAD_ARGUMENT;
    auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    const bool vec = E % 4 == 0 && part_stride % 4 == 0 && al(h) && al(a) && al(wb) && al(w) && al(out);
    AIR_DISPATCH(out_dtype, TO, {
        auto go = [&](auto kernel) {
            if (smem > 48 * 1024) {
                cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (err != cudaSuccess) return (int)err;
            }
            return air::launch(kernel, R, threads, smem, stream, h, a, a_parts, (size_t)part_stride, wb, eps_b, w,
                               (TO*)out, rows, E, eps);
        };
        return vec ? go(air::normed_add_norm_kernel<TO, true>) : go(air::normed_add_norm_kernel<TO, false>);
    });
    return 0;
}

AIR_API int air_relu2(const void* in, int in_dtype, void* out, int out_dtype, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    const int vec = total % 4 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0;
    const long long items = vec ? total / 4 : total;
    const int blocks = (int)((items + 255) / 256 < 148 * 16 ? (items + 255) / 256 : 148 * 16);
    AIR_DISPATCH(in_dtype, TI, AIR_DISPATCH(out_dtype, TO,
        return air::launch(air::relu2_kernel<TI, TO>, blocks, 256, 0, stream, (const TI*)in, (TO*)out, (size_t)total,
                           vec)));
    return 0;
}

AIR_API int air_sigmoid_gate(void* x, int dtype, const float* gate, int ldg, const int* token_seq, int T, int C,
                             cudaStream_t stream) {
    if (T <= 0 || C <= 0) return 0;
    const long long total = (long long)T * C;
    const int vec = C % 4 == 0 && ldg % 4 == 0 && (((uintptr_t)x | (uintptr_t)gate) & 15) == 0;
    const long long items = vec ? total / 4 : total;
    const int blocks = (int)((items + 255) / 256 < 148 * 16 ? (items + 255) / 256 : 148 * 16);
    AIR_DISPATCH(dtype, TX, return air::launch(air::sigmoid_gate_kernel<TX>, blocks, 256, 0, stream, (TX*)x, gate, ldg,
                                               token_seq, C, (size_t)total, vec));
    return 0;
}

AIR_API int air_trace_set_sandwich_ops(unsigned long long* buffer) { return air::set_trace_here(buffer); }
