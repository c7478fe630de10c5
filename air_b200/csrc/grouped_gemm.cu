// Matrix products in groups: C_g = A_g W_g^T for many g in one launch, where every group has a matrix W_g [N, K] of its
// own and a list of rows.  Two users: the experts of a mixture (group = expert, its rows are the tokens that chose it,
// known only on the device) and products per head (group = head, every group has all the step's rows).
//
//   Rows.  A group's rows are consecutive *slots*.  With `start` (device, [G + 1]) group g has the slots start[g] ..
//   start[g + 1], and `tiles` (device: pairs (group, first slot), their number in num_tiles) says which row tiles
//   exist; a block whose index is beyond that number leaves.  Without `start` every group has rows_per_group rows
//   and the grid is (column tiles, row tiles, groups).
//   Where a slot's row of A lies: with a_index, row a_index[slot] / a_div, times a_scale[a_index[slot]] if a_scale is
//   given (the product is rounded to A's type, as if a scaled copy of the row had been made); else row `slot`, or
//   with a_local the row slot - (the group's first slot); plus g * a_group_stride elements.
//   Where a slot's row of C goes: with o_index, p = o_index[slot]: part p % o_div, row p / o_div of out
//   [o_div, rows, N] (o_part_stride elements per part); else row `slot` (or, o_local, the row inside the group) plus
//   g * o_group_stride.  With o_scale the row of C is multiplied, in 32-bit before it is written, by
//   o_scale[o_index[slot]] (the weight of a token's choice on the expert's OUTPUT) or, without o_index, by
//   o_scale[row * o_scale_ld + g] (a gate per token and head behind a product per head).
//   Epilogue 0: C as float32 or in A's type.  Epilogue 1: W_g is [2 F, K], blocks of gate_block rows of the gate and
//   as many of the linear branch in turn (gate_block = F: all gate rows, then all linear rows), the arrangement that
//   the dense gated feed-forward uses; C [rows, F] = silu(gate) * linear in A's type.  Epilogue 2: C = max(x, 0)^2 of the
//   plain product x, in A's type (the hidden layer of an expert without a gate).
//
// Arithmetic.  float32 operands (and bfloat16 ones whose strides are not multiples of 8 elements): 32-bit multiply-adds
// on the CUDA cores, k ascending; a tile is 64 x 64, a thread holds 4 x 4 of it (grouped_gemm_kernel).  bfloat16
// operands: the warp-level tensor-core instruction (m16n8k16, 32-bit accumulators), four warps of 16 rows by 64
// columns each, operands brought into a ring of four shared-memory stages by cp.async in steps of 32 of k
// (grouped_gemm_tc_kernel).  Either way a row's result depends on nothing but the row and W_g.
#include "common.cuh"
#include "mma.cuh"

namespace air {

struct GroupedArgs {
    const void* A; long long lda; long long a_group_stride; const int* a_index; int a_div; int a_local;
    const float* a_scale;
    const void* W; long long w_group_stride;
    void* out; long long ldo; long long o_group_stride; const int* o_index; int o_div; long long o_part_stride;
    int o_local; int out_f32;
    const int* start; int rows_per_group; const int* tiles; const int* num_tiles;
    int N, K;
    int gate_block;      // epilogue 1: rows of W_g come in blocks of gate_block gate rows and as many linear rows in turn
    const float* o_scale; int o_scale_ld;
};

constexpr int GG_BM = 64, GG_BN = 64, GG_BK = 16;

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(const GroupedArgs p) {
    __shared__ float As[GG_BK][GG_BM + 4];
    __shared__ float Ws[EPI == 1 ? 2 : 1][GG_BK][GG_BN + 4];
    __shared__ long long a_off[GG_BM], o_off[GG_BM];
    __shared__ float a_mul[GG_BM], o_mul[GG_BM];
    pdl_enter(TR_GROUPED_GEMM);
    int g, slot0, first, rows;
    if (p.start) {
        if ((int)blockIdx.y >= *p.num_tiles) return;
        g = p.tiles[2 * blockIdx.y];
        slot0 = p.tiles[2 * blockIdx.y + 1];
        first = p.start[g];
        rows = min(GG_BM, p.start[g + 1] - slot0);
    } else {
        g = blockIdx.z;
        first = g * p.rows_per_group;
        slot0 = first + blockIdx.y * GG_BM;
        rows = min(GG_BM, p.rows_per_group - (int)blockIdx.y * GG_BM);
    }
    if (rows <= 0) return;
    const int n0 = blockIdx.x * GG_BN;
    const int tid = threadIdx.x;
    if (tid < GG_BM) {
        long long a = -1, o = -1;
        float mul = 1.f, omul = 1.f;
        if (tid < rows) {
            const int slot = slot0 + tid;
            if (p.a_index) {
                const int src = p.a_index[slot];
                a = (long long)(src / p.a_div) * p.lda + (long long)g * p.a_group_stride;
                if (p.a_scale) mul = p.a_scale[src];
            } else {
                a = (long long)(p.a_local ? slot - first : slot) * p.lda + (long long)g * p.a_group_stride;
            }
            if (p.o_index) {
                const int dst = p.o_index[slot];
                o = (long long)(dst % p.o_div) * p.o_part_stride + (long long)(dst / p.o_div) * p.ldo;
                if (p.o_scale) omul = p.o_scale[dst];
            } else {
                o = (long long)(p.o_local ? slot - first : slot) * p.ldo + (long long)g * p.o_group_stride;
                if (p.o_scale) omul = p.o_scale[(long long)(p.o_local ? slot - first : slot) * p.o_scale_ld + g];
            }
        }
        a_off[tid] = a;
        o_off[tid] = o;
        a_mul[tid] = mul;
        o_mul[tid] = omul;
    }
    __syncthreads();
    const T* A = (const T*)p.A;
    const T* W = (const T*)p.W + (size_t)g * p.w_group_stride;
    const int N = p.N, K = p.K;
    const int lm = tid >> 2, lk = (tid & 3) * 4;      // what this thread loads: row lm, k lk .. lk + 3
    const int ty = tid >> 4, tx = tid & 15;
    float acc[EPI == 1 ? 2 : 1][4][4];
#pragma unroll
    for (int e = 0; e < (EPI == 1 ? 2 : 1); ++e)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[e][i][j] = 0.f;
    const long long arow = a_off[lm];
    const float amul = a_mul[lm];
    const bool scaled = p.a_scale != nullptr;
    for (int k0 = 0; k0 < K; k0 += GG_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            float a = 0.f;
            if (arow >= 0 && k < K) {
                a = to_float(A[arow + k]);
                if (scaled) a = to_float(from_float<T>(a * amul));
            }
            As[lk + i][lm] = a;
#pragma unroll
            for (int e = 0; e < (EPI == 1 ? 2 : 1); ++e) {
                const int n = n0 + lm;
                const size_t wrow = EPI == 1 ? (size_t)(n / p.gate_block) * 2 * p.gate_block + e * p.gate_block + n % p.gate_block : n;
                Ws[e][lk + i][lm] = (n < N && k < K) ? to_float(W[wrow * K + k]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GG_BK; ++kk) {
            float a[4], b[EPI == 1 ? 2 : 1][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int e = 0; e < (EPI == 1 ? 2 : 1); ++e)
#pragma unroll
                for (int j = 0; j < 4; ++j) b[e][j] = Ws[e][kk][tx * 4 + j];
#pragma unroll
            for (int e = 0; e < (EPI == 1 ? 2 : 1); ++e)
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[e][i][j] = fmaf(a[i], b[e][j], acc[e][i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long o = o_off[ty * 4 + i];
        if (o < 0) continue;
        const float om = o_mul[ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (EPI == 1) {
                const float gate = acc[0][i][j], lin = acc[EPI == 1 ? 1 : 0][i][j];
                ((T*)p.out)[o + n] = from_float<T>(gate / (1.f + expf(-gate)) * lin);
            } else if (EPI == 2) {
                const float r = fmaxf(acc[0][i][j], 0.f);
                ((T*)p.out)[o + n] = from_float<T>(r * r);
            } else if (p.out_f32) {
                ((float*)p.out)[o + n] = acc[0][i][j] * om;
            } else {
                ((T*)p.out)[o + n] = from_float<T>(acc[0][i][j] * om);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------- bfloat16, tensor cores
constexpr int GT_BK = 32, GT_LD = GT_BK + 8;      // a row of a staged tile: 32 elements and 16 bytes of padding
constexpr int GT_STAGES = 4;                      // steps of k in flight: a step of few rows is a stream of weights

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src, bool valid) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;             // 0: the 16 bytes are zero-filled, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t scaled_pair(uint32_t word, float m) {
    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&word);
    return pack_bf16(__low2float(x) * m, __high2float(x) * m);
}

template <int EPI>
__global__ void __launch_bounds__(128)
grouped_gemm_tc_kernel(const GroupedArgs p) {
    constexpr int NW = EPI == 1 ? 2 : 1;
    constexpr int TILE = GG_BM * GT_LD;           // elements of one staged tile
    extern __shared__ __align__(16) __nv_bfloat16 staged[];      // [stages][1 + NW][64][GT_LD]
    __shared__ long long a_off[GG_BM], o_off[GG_BM];
    __shared__ float a_mul[GG_BM], o_mul[GG_BM];
    pdl_enter(TR_GROUPED_GEMM);
    int g, slot0, first, rows;
    if (p.start) {
        if ((int)blockIdx.y >= *p.num_tiles) return;
        g = p.tiles[2 * blockIdx.y];
        slot0 = p.tiles[2 * blockIdx.y + 1];
        first = p.start[g];
        rows = min(GG_BM, p.start[g + 1] - slot0);
    } else {
        g = blockIdx.z;
        first = g * p.rows_per_group;
        slot0 = first + blockIdx.y * GG_BM;
        rows = min(GG_BM, p.rows_per_group - (int)blockIdx.y * GG_BM);
    }
    if (rows <= 0) return;
    const int n0 = blockIdx.x * GG_BN;
    const int tid = threadIdx.x;
    if (tid < GG_BM) {
        long long a = -1, o = -1;
        float mul = 1.f, omul = 1.f;
        if (tid < rows) {
            const int slot = slot0 + tid;
            if (p.a_index) {
                const int src = p.a_index[slot];
                a = (long long)(src / p.a_div) * p.lda + (long long)g * p.a_group_stride;
                if (p.a_scale) mul = p.a_scale[src];
            } else {
                a = (long long)(p.a_local ? slot - first : slot) * p.lda + (long long)g * p.a_group_stride;
            }
            if (p.o_index) {
                const int dst = p.o_index[slot];
                o = (long long)(dst % p.o_div) * p.o_part_stride + (long long)(dst / p.o_div) * p.ldo;
                if (p.o_scale) omul = p.o_scale[dst];
            } else {
                o = (long long)(p.o_local ? slot - first : slot) * p.ldo + (long long)g * p.o_group_stride;
                if (p.o_scale) omul = p.o_scale[(long long)(p.o_local ? slot - first : slot) * p.o_scale_ld + g];
            }
        }
        a_off[tid] = a;
        o_off[tid] = o;
        a_mul[tid] = mul;
        o_mul[tid] = omul;
    }
    __syncthreads();
    const __nv_bfloat16* A = (const __nv_bfloat16*)p.A;
    const __nv_bfloat16* W = (const __nv_bfloat16*)p.W + (size_t)g * p.w_group_stride;
    const int N = p.N, K = p.K;
    const bool scaled = p.a_scale != nullptr;
    // what this thread brings per step: chunks (16 bytes, 8 of k) tid and tid + 128 of the 64 x 4 chunks of every tile
    const __nv_bfloat16* src_a[2];
    const __nv_bfloat16* src_w[NW][2];
    int dst_at[2], kc_of[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c = tid + 128 * i, row = c >> 2;
        kc_of[i] = (c & 3) * 8;
        dst_at[i] = row * GT_LD + kc_of[i];
        src_a[i] = a_off[row] >= 0 ? A + a_off[row] + kc_of[i] : nullptr;
#pragma unroll
        for (int e = 0; e < NW; ++e) {
            const int n = n0 + row;
            const size_t wrow = EPI == 1 ? (size_t)(n / p.gate_block) * 2 * p.gate_block + e * p.gate_block + n % p.gate_block : n;
            src_w[e][i] = n < N ? W + wrow * K + kc_of[i] : nullptr;
        }
    }
    auto bring = [&](int stage, int k0) {
        __nv_bfloat16* base = staged + (size_t)stage * (1 + NW) * TILE;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const bool in_k = k0 + kc_of[i] < K;
            cp_async16(base + dst_at[i], src_a[i] ? src_a[i] + k0 : (const __nv_bfloat16*)A, in_k && src_a[i]);
#pragma unroll
            for (int e = 0; e < NW; ++e)
                cp_async16(base + (1 + e) * TILE + dst_at[i], src_w[e][i] ? src_w[e][i] + k0 : W, in_k && src_w[e][i]);
        }
    };
    const int warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
    const int r0 = warp * 16;
    const float m_lo = a_mul[r0 + gq], m_hi = a_mul[r0 + gq + 8];
    float acc[NW][8][4];
#pragma unroll
    for (int e = 0; e < NW; ++e)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[e][j][i] = 0.f;
    const int steps = (K + GT_BK - 1) / GT_BK;
#pragma unroll
    for (int s = 0; s < GT_STAGES - 1; ++s) {
        if (s < steps) bring(s, s * GT_BK);
        cp_async_commit();
    }
    for (int step = 0; step < steps; ++step) {
        cp_async_wait<GT_STAGES - 2>();           // this step's tiles have landed (for this thread's copies)
        __syncthreads();                          // ... for everybody's, and the stage refilled below has been read
        if (step + GT_STAGES - 1 < steps) bring((step + GT_STAGES - 1) % GT_STAGES, (step + GT_STAGES - 1) * GT_BK);
        cp_async_commit();
        const __nv_bfloat16* As = staged + (size_t)(step % GT_STAGES) * (1 + NW) * TILE;
        if (r0 >= rows) continue;                 // a warp whose 16 rows are all beyond the tile's (a step of few tokens
                                                  // has one or two rows per expert) only helps to bring the weights
#pragma unroll
        for (int kk = 0; kk < GT_BK; kk += 16) {
            uint32_t a0 = *reinterpret_cast<const uint32_t*>(As + (r0 + gq) * GT_LD + kk + 2 * tq);
            uint32_t a1 = *reinterpret_cast<const uint32_t*>(As + (r0 + gq + 8) * GT_LD + kk + 2 * tq);
            uint32_t a2 = *reinterpret_cast<const uint32_t*>(As + (r0 + gq) * GT_LD + kk + 2 * tq + 8);
            uint32_t a3 = *reinterpret_cast<const uint32_t*>(As + (r0 + gq + 8) * GT_LD + kk + 2 * tq + 8);
            if (scaled) {      // the weight of the row's choice, rounded as a scaled copy of the row would be
                a0 = scaled_pair(a0, m_lo); a2 = scaled_pair(a2, m_lo);
                a1 = scaled_pair(a1, m_hi); a3 = scaled_pair(a3, m_hi);
            }
#pragma unroll
            for (int e = 0; e < NW; ++e) {
                const __nv_bfloat16* Ws = As + (1 + e) * TILE;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(Ws + (8 * j + gq) * GT_LD + kk + 2 * tq);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(Ws + (8 * j + gq) * GT_LD + kk + 2 * tq + 8);
                    mma_bf16_16816(acc[e][j], a0, a1, a2, a3, b0, b1);
                }
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const long long o = o_off[r0 + gq + 8 * half];
        if (o < 0) continue;
        const float om = o_mul[r0 + gq + 8 * half];
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int n = n0 + 8 * j + 2 * tq + i;
                if (n >= N) continue;
                const float v = acc[0][j][2 * half + i] * (EPI == 0 ? om : 1.f);
                if (EPI == 1) {
                    const float lin = acc[NW - 1][j][2 * half + i];
                    ((__nv_bfloat16*)p.out)[o + n] = __float2bfloat16_rn(v / (1.f + expf(-v)) * lin);
                } else if (EPI == 2) {
                    const float r = fmaxf(acc[0][j][2 * half + i], 0.f);
                    ((__nv_bfloat16*)p.out)[o + n] = __float2bfloat16_rn(r * r);
                } else if (p.out_f32) {
                    ((float*)p.out)[o + n] = v;
                } else {
                    ((__nv_bfloat16*)p.out)[o + n] = __float2bfloat16_rn(v);
                }
            }
    }
}

}  // namespace air

AIR_API int air_grouped_gemm(const void* A, long long lda, long long a_group_stride, const int* a_index, int a_div,
                             int a_local, const float* a_scale, const void* W, long long w_group_stride, void* out,
                             long long ldo, long long o_group_stride, const int* o_index, int o_div,
                             long long o_part_stride, int o_local, int out_f32, const int* start, int rows_per_group,
                             const int* tiles, const int* num_tiles, int max_tiles, int groups, int N, int K,
                             int dtype, int epi, int gate_block, const float* o_scale, int o_scale_ld,
                             cudaStream_t stream) {
    if (N <= 0 || K <= 0 || groups <= 0) return 0;
    if ((start != nullptr) != (tiles != nullptr) || (start && !num_tiles) || epi < 0 || epi > 2 ||
        (a_index && a_div <= 0) || (o_index && o_div <= 0) || (a_scale && !a_index) || (o_scale && epi))
        return AIR_ERR_BAD_ARGUMENT;
    if (epi == 1 && gate_block <= 0) gate_block = N;
    if (epi == 1 && N % gate_block) return AIR_ERR_BAD_ARGUMENT;
    air::GroupedArgs p{A, lda, a_group_stride, a_index, a_div, a_local, a_scale, W, w_group_stride, out, ldo,
                       o_group_stride, o_index, o_div, o_part_stride, o_local, out_f32, start, rows_per_group, tiles,
                       num_tiles, N, K, gate_block, o_scale, o_scale_ld};
    const int row_tiles = start ? max_tiles : (rows_per_group + air::GG_BM - 1) / air::GG_BM;
    if (row_tiles <= 0) return 0;
    if (row_tiles > 65535 || groups > 65535) return AIR_ERR_BAD_ARGUMENT;
    dim3 grid((N + air::GG_BN - 1) / air::GG_BN, row_tiles, start ? 1 : groups);
    // the tensor-core kernel fetches 8 elements at a time: every row of A and of W must start on 16 bytes
    const bool aligned = K % 8 == 0 && lda % 8 == 0 && a_group_stride % 8 == 0 && ((uintptr_t)A & 15) == 0 &&
                         ((uintptr_t)W & 15) == 0;
    if (dtype == AIR_BF16 && aligned) {
        const size_t smem = (size_t)air::GT_STAGES * (epi == 1 ? 3 : 2) * air::GG_BM * air::GT_LD * 2;
        if (epi == 1) {
            cudaFuncSetAttribute(air::grouped_gemm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            return air::launch(air::grouped_gemm_tc_kernel<1>, grid, 128, smem, stream, p);
        }
        if (epi == 2) return air::launch(air::grouped_gemm_tc_kernel<2>, grid, 128, smem, stream, p);
        return air::launch(air::grouped_gemm_tc_kernel<0>, grid, 128, smem, stream, p);
    }
    AIR_DISPATCH(dtype, TT, {
        if (epi == 1) return air::launch(air::grouped_gemm_kernel<TT, 1>, grid, 256, 0, stream, p);
        if (epi == 2) return air::launch(air::grouped_gemm_kernel<TT, 2>, grid, 256, 0, stream, p);
        return air::launch(air::grouped_gemm_kernel<TT, 0>, grid, 256, 0, stream, p);
    });
    return 0;
}

AIR_API int air_trace_set_grouped_gemm(unsigned long long* buffer) { return air::set_trace_here(buffer); }
