// Two row-wise operations of blocks whose sub-layers stand side by side and of gated feed-forwards with limits.
//
//   glu_kernel          out[t, i] = g' * sigmoid(alpha * g') * (u' + shift), with g' = min(gate, limit) and
//                       u' = clamp(up, -limit, limit) where limit > 0 (else gate and up as they are).  alpha = 1,
//                       shift = 0, limit = 0 is SiLU(gate) * up.  The input [T, 2I] holds blocks of `block` gate
//                       columns and `block` up columns in turn.
//   head_gate_kernel    x[t, h, :] *= gate[t, h], for attention kernels that do not multiply by a gate as they write
//   scaled_norm_kernel  x = h + sa * a + sb * b (float32; a scale per column, each term optional; a term may come as
//                       the partial sums of a split product, [parts, T, E], which are added in order), written back into
//                       the stream h when no rows are named, and out = x / sqrt(mean(x^2) + eps) * w.  With `rows`
//                       the kernel reads h[rows[r]] and leaves h alone.  Without w it only completes the stream.
//   polynorm_kernel     z = in[t, :] + bias; out[t, i] = a z_i / r1 + b z_i^2 / r2 + c z_i^3 / r3 + e with r_p = sqrt(mean_i(z_i^(2p))
//                       + eps) over the row's F columns; 32-bit, written in out's type.  out has
//                       ldo >= F columns: column F (if any) receives 1 and the ones behind it 0, so that a product
//                       whose matrix holds a bias in column F adds that bias.  polynorm_rows_kernel is the same with
//                       the row in registers (rows that eight accesses of four columns per thread cover).
#include "common.cuh"

namespace air {

// The three sums over the block and, from them, the three factors a / r1, b / r2, c / r3: the first warp adds the
// warps' sums (in an order that depends on the block's size only) and takes roots and quotients once for the block.
__device__ __forceinline__ void polynorm_factors(float s2, float s4, float s6, float (*scratch)[32], int F, float a,
                                                 float b, float c, float eps, float& r1, float& r2, float& r3) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    s2 = warp_sum(s2); s4 = warp_sum(s4); s6 = warp_sum(s6);
    if (lane == 0) { scratch[0][warp] = s2; scratch[1][warp] = s4; scratch[2][warp] = s6; }
    __syncthreads();
    if (warp == 0) {
        s2 = warp_sum(lane < warps ? scratch[0][lane] : 0.f);
        s4 = warp_sum(lane < warps ? scratch[1][lane] : 0.f);
        s6 = warp_sum(lane < warps ? scratch[2][lane] : 0.f);
        if (lane == 0) {
            scratch[0][0] = a / sqrtf(s2 / (float)F + eps);
            scratch[1][0] = b / sqrtf(s4 / (float)F + eps);
            scratch[2][0] = c / sqrtf(s6 / (float)F + eps);
        }
    }
    __syncthreads();
    r1 = scratch[0][0]; r2 = scratch[1][0]; r3 = scratch[2][0];
}

// A block per row.  The row (with its bias) is kept in shared memory between the pass that takes the three sums of
// squares and the pass that writes (ROW_IN_SMEM; rows too long for that are read again), four elements at a time
// where the row's start and length allow (VEC).  Few rows (a decode step) get blocks of 1,024 threads, so that all of
// a row's loads are under way at once.
template <typename TO, bool VEC, bool ROW_IN_SMEM>
__global__ void __launch_bounds__(1024)
polynorm_kernel(const float* __restrict__ in, int ld, const float* __restrict__ bias, TO* __restrict__ out, int ldo,
                int F, float a, float b, float c, float e, float eps) {
    __shared__ float scratch[3][32];
    extern __shared__ __align__(16) float zrow[];
    pdl_enter(TR_POLYNORM);
    const int t = blockIdx.x;
    const float* row = in + (size_t)t * ld;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    auto take = [&](float z) {
        const float z2 = z * z;
        s2 += z2;
        s4 = fmaf(z2, z2, s4);
        s6 = fmaf(z2 * z, z2 * z, s6);
    };
    if (VEC) {
        // four accesses of a thread are issued before the first is used (the sums are taken in the order of the columns
        // all the same): with one access under way per thread a block keeps too few bytes in flight to fill the memory
        constexpr int U = 4;
        const int step = blockDim.x * 4;
        int i = threadIdx.x * 4;
        for (; i + (U - 1) * step < F; i += U * step) {
            float z[U][4], bv[U][4];
#pragma unroll
            for (int u = 0; u < U; ++u) load4(row + i + u * step, z[u]);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (bias) load4(bias + i + u * step, bv[u]);
                else bv[u][0] = bv[u][1] = bv[u][2] = bv[u][3] = 0.f;
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    z[u][j] += bv[u][j];
                    take(z[u][j]);
                }
                if (ROW_IN_SMEM) store4(zrow + i + u * step, z[u]);
            }
        }
        for (; i < F; i += step) {
            float z[4], bv[4] = {0.f, 0.f, 0.f, 0.f};
            load4(row + i, z);
            if (bias) load4(bias + i, bv);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                z[j] += bv[j];
                take(z[j]);
            }
            if (ROW_IN_SMEM) store4(zrow + i, z);
        }
    } else {
        for (int i = threadIdx.x; i < F; i += blockDim.x) {
            const float z = row[i] + (bias ? bias[i] : 0.f);
            take(z);
            if (ROW_IN_SMEM) zrow[i] = z;
        }
    }
    float r1, r2, r3;
    polynorm_factors(s2, s4, s6, scratch, F, a, b, c, eps, r1, r2, r3);
    TO* dst = out + (size_t)t * ldo;
    auto act = [&](float z) {
        const float z2 = z * z;
        return z * r1 + z2 * r2 + z2 * z * r3 + e;
    };
    if (VEC) {
        for (int i = threadIdx.x * 4; i < F; i += blockDim.x * 4) {
            float z[4], bv[4] = {0.f, 0.f, 0.f, 0.f};
            if (ROW_IN_SMEM) {
                load4(zrow + i, z);
            } else {
                load4(row + i, z);
                if (bias) load4(bias + i, bv);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) z[j] = act(z[j] + bv[j]);
            store4(dst + i, z);
        }
    } else {
        for (int i = threadIdx.x; i < F; i += blockDim.x)
            dst[i] = from_float<TO>(act(ROW_IN_SMEM ? zrow[i] : row[i] + (bias ? bias[i] : 0.f)));
    }
    for (int i = F + threadIdx.x; i < ldo; i += blockDim.x) dst[i] = from_float<TO>(i == F ? 1.f : 0.f);
}

// The same with the row in registers: K accesses of four columns per thread, all issued before the first is used, for
// rows of up to 4 K blockDim columns (row start and length multiples of 4).  The sums are taken in the order of the
// other form (a thread's columns ascending, then the block's warps in order).
template <typename TO, int K>
__global__ void __launch_bounds__(K > 4 ? 512 : 1024)
polynorm_rows_kernel(const float* __restrict__ in, int ld, const float* __restrict__ bias, TO* __restrict__ out, int ldo,
                     int F, float a, float b, float c, float e, float eps) {
    __shared__ float scratch[3][32];
    pdl_enter(TR_POLYNORM);
    const int t = blockIdx.x;
    const float* row = in + (size_t)t * ld;
    const int step = blockDim.x * 4;
    float z[K][4];
#pragma unroll
    for (int k = 0; k < K; ++k) {
        const int i = threadIdx.x * 4 + k * step;
        if (i < F) load4(row + i, z[k]);
        else z[k][0] = z[k][1] = z[k][2] = z[k][3] = 0.f;
    }
    if (bias) {
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int i = threadIdx.x * 4 + k * step;
            float bv[4];
            if (i < F) {
                load4(bias + i, bv);
#pragma unroll
                for (int j = 0; j < 4; ++j) z[k][j] += bv[j];
            }
        }
    }
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
        if (threadIdx.x * 4 + k * step < F) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float z2 = z[k][j] * z[k][j];
                s2 += z2;
                s4 = fmaf(z2, z2, s4);
                s6 = fmaf(z2 * z[k][j], z2 * z[k][j], s6);
            }
        }
    }
    float r1, r2, r3;
    polynorm_factors(s2, s4, s6, scratch, F, a, b, c, eps, r1, r2, r3);
    TO* dst = out + (size_t)t * ldo;
#pragma unroll
    for (int k = 0; k < K; ++k) {
        const int i = threadIdx.x * 4 + k * step;
        if (i < F) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float v = z[k][j], v2 = v * v;
                z[k][j] = v * r1 + v2 * r2 + v2 * v * r3 + e;
            }
            store4(dst + i, z[k]);
        }
    }
    for (int i = F + threadIdx.x; i < ldo; i += blockDim.x) dst[i] = from_float<TO>(i == F ? 1.f : 0.f);
}

template <typename TI, typename TO>
__global__ void glu_kernel(const TI* __restrict__ in, TO* __restrict__ out, int I, int block, size_t total,
                           float alpha, float limit, float shift) {
    pdl_enter(TR_GLU);
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I;
        const int i = (int)(idx % I);
        const TI* row = in + t * 2 * (size_t)I + (size_t)(i / block) * 2 * block;
        float g = to_float(row[i % block]), u = to_float(row[block + i % block]);
        if (limit > 0.f) {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
        }
        out[idx] = from_float<TO>(g / (1.f + expf(-alpha * g)) * (u + shift));
    }
}

// x [T, H, d] *= gate[T, H] in place (one gate per token and head); rows whose token_seq is negative are padding.
template <typename TX>
__global__ void head_gate_kernel(TX* __restrict__ x, const float* __restrict__ gate, const int* __restrict__ token_seq,
                                 int H, int d, size_t total) {
    pdl_enter(TR_HEAD_GATE);
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t th = idx / d;
        if (token_seq[th / H] < 0) continue;
        x[idx] = from_float<TX>(to_float(x[idx]) * gate[th]);
    }
}

// VEC: four columns per access (E and the parts' stride multiples of 4, all pointers on 16-byte boundaries).
template <typename TW, typename TO, bool VEC>
__global__ void scaled_norm_kernel(float* __restrict__ h, const float* __restrict__ a, const float* __restrict__ sa,
                                   int a_parts, const float* __restrict__ b, const float* __restrict__ sb, int b_parts,
                                   size_t part_stride, const TW* __restrict__ w, TO* __restrict__ out,
                                   const int* __restrict__ rows, int E, float eps) {
    __shared__ float scratch[32];
    extern __shared__ __align__(16) float xrow[];
    pdl_enter(TR_SCALED_NORM);
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * E;
    const bool keep = !rows && (a || b);
    float ss = 0.f;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
            float x[4], t[4], u[4], sc[4];
            load4(h + src + i, x);
            if (a) {
                load4(a + src + i, t);
#pragma unroll 4
                for (int p = 1; p < a_parts; ++p) {                                   // (loads ahead, sums in order)
                    load4(a + p * part_stride + src + i, u);
#pragma unroll
                    for (int j = 0; j < 4; ++j) t[j] += u[j];
                }
                if (sa) load4(sa + i, sc);
#pragma unroll
                for (int j = 0; j < 4; ++j) x[j] += (sa ? sc[j] : 1.f) * t[j];
            }
            if (b) {
                load4(b + src + i, t);
#pragma unroll 4
                for (int p = 1; p < b_parts; ++p) {
                    load4(b + p * part_stride + src + i, u);
#pragma unroll
                    for (int j = 0; j < 4; ++j) t[j] += u[j];
                }
                if (sb) load4(sb + i, sc);
#pragma unroll
                for (int j = 0; j < 4; ++j) x[j] += (sb ? sc[j] : 1.f) * t[j];
            }
            store4(xrow + i, x);
#pragma unroll
            for (int j = 0; j < 4; ++j) ss += x[j] * x[j];
            if (keep) store4(h + src + i, x);
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            float x = h[src + i];
            if (a) {
                float t = a[src + i];
#pragma unroll 4
                for (int p = 1; p < a_parts; ++p) t += a[p * part_stride + src + i];
                x += (sa ? sa[i] : 1.f) * t;
            }
            if (b) {
                float t = b[src + i];
#pragma unroll 4
                for (int p = 1; p < b_parts; ++p) t += b[p * part_stride + src + i];
                x += (sb ? sb[i] : 1.f) * t;
            }
            xrow[i] = x;
            ss += x * x;
            if (keep) h[src + i] = x;
        }
    }
    if (!w) return;
    const float total = block_sum(ss, scratch);
    const float scale = rsqrtf(total / (float)E + eps);
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
            out[(size_t)r * E + i] = from_float<TO>(xrow[i] * scale * to_float(w[i]));
    }
}

}  // namespace air

AIR_API int air_glu(const void* in, int in_dtype, void* out, int out_dtype, int T, int I, int block, float alpha,
                    float limit, float shift, cudaStream_t stream) {
    const size_t total = (size_t)T * I;
    if (total == 0) return 0;
    if (block <= 0 || I % block) return AIR_ERR_BAD_ARGUMENT;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    AIR_DISPATCH(in_dtype, TI, AIR_DISPATCH(out_dtype, TO, {
        return air::launch(air::glu_kernel<TI, TO>, blocks, 256, 0, stream, (const TI*)in, (TO*)out, I, block, total,
                           alpha, limit, shift);
    }));
    return 0;
}

AIR_API int air_polynorm(const float* in, int ld, const float* bias, void* out, int out_dtype, int ldo, int T, int F,
                         float a, float b, float c, float e, float eps, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (F <= 0 || ldo < F || ld < F) return AIR_ERR_BAD_ARGUMENT;
    const int threads = T <= 296 ? 1024 : 256;
    const bool vec = F % 4 == 0 && ld % 4 == 0 && ldo % 4 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
                     (!bias || ((uintptr_t)bias & 15) == 0);
    if (vec) {
        // the row in registers: the fewest accesses per thread (1, 2, 4, 8) with which a block of at most `most` threads
        // covers the row
        // (many rows: narrow blocks where eight accesses a thread cover the row, so that an SM holds four blocks in
        // different phases; few rows: wide blocks, so that a row's loads are all under way at once)
        const int f4 = F / 4;
        const int most = T <= 296 ? 1024 : ((f4 + 7) / 8 <= 256 ? 256 : 512);
        for (int k = 1; k <= 8; k *= 2) {
            if ((f4 + k - 1) / k > (k > 4 && most > 512 ? 512 : most)) continue;
            int th = ((f4 + k - 1) / k + 31) / 32 * 32;
            if (th < 128) th = 128;
            AIR_DISPATCH(out_dtype, TO, {
                auto run = [&](auto kernel) {
                    return air::launch(kernel, T, th, 0, stream, in, ld, bias, (TO*)out, ldo, F, a, b, c, e, eps);
                };
                if (k == 1) return run(air::polynorm_rows_kernel<TO, 1>);
                if (k == 2) return run(air::polynorm_rows_kernel<TO, 2>);
                if (k == 4) return run(air::polynorm_rows_kernel<TO, 4>);
                return run(air::polynorm_rows_kernel<TO, 8>);
            });
        }
    }
    const size_t row_bytes = sizeof(float) * (size_t)F;
    const bool in_smem = row_bytes <= 160 * 1024;
    const size_t smem = in_smem ? row_bytes : 0;
    AIR_DISPATCH(out_dtype, TO, {
        auto go = [&](auto kernel) {
            if (smem > 48 * 1024) {
                cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (err != cudaSuccess) return (int)err;
            }
            return air::launch(kernel, T, threads, smem, stream, in, ld, bias, (TO*)out, ldo, F, a, b, c, e, eps);
        };
        if (vec) return in_smem ? go(air::polynorm_kernel<TO, true, true>) : go(air::polynorm_kernel<TO, true, false>);
        return in_smem ? go(air::polynorm_kernel<TO, false, true>) : go(air::polynorm_kernel<TO, false, false>);
    });
    return 0;
}

AIR_API int air_head_gate(void* x, int dtype, const float* gate, const int* token_seq, int T, int H, int d,
                          cudaStream_t stream) {
    const size_t total = (size_t)T * H * d;
    if (total == 0) return 0;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    AIR_DISPATCH(dtype, TX, return air::launch(air::head_gate_kernel<TX>, blocks, 256, 0, stream, (TX*)x, gate, token_seq,
                                               H, d, total));
    return 0;
}

AIR_API int air_scaled_norm(float* h, const float* a, const float* sa, int a_parts, const float* b, const float* sb,
                            int b_parts, long long part_stride, const void* w, int w_dtype, void* out, int out_dtype,
                            const int* rows, int R, int E, float eps, cudaStream_t stream) {
    if (R <= 0) return 0;
    // few rows: a block as wide as half a row, so that a row's loads are all under way at once
    int threads = E >= 1024 ? 256 : 128;
    if (R <= 256) threads = E / 2 >= 1024 ? 1024 : (E / 2 > threads ? (E / 2 + 31) / 32 * 32 : threads);
    const size_t smem = sizeof(float) * (size_t)E;
    if (smem > 200 * 1024) return AIR_ERR_BAD_ARGUMENT;
    auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    const bool vec = E % 4 == 0 && part_stride % 4 == 0 && al(h) && al(a) && al(sa) && al(b) && al(sb) && al(w) && al(out);
    AIR_DISPATCH(w_dtype, TW, AIR_DISPATCH(out_dtype, TO, {
        auto go = [&](auto kernel) {
            if (smem > 48 * 1024) {
                cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (err != cudaSuccess) return (int)err;
            }
            return air::launch(kernel, R, threads, smem, stream, h, a, sa, a_parts, b, sb, b_parts, (size_t)part_stride,
                               (const TW*)w, (TO*)out, rows, E, eps);
        };
        return vec ? go(air::scaled_norm_kernel<TW, TO, true>) : go(air::scaled_norm_kernel<TW, TO, false>);
    }));
    return 0;
}

AIR_API int air_trace_set_gated_ops(unsigned long long* buffer) { return air::set_trace_here(buffer); }
