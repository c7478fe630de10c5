// Paged attention with 32-bit arithmetic in which a block serves all the query heads that share a key/value head, so
// that a key and its value are read from memory once for the whole group: the kernel of single next tokens and short
// portions for layers whose keys the tile kernels do not take (a latent row per token that every head reads, keys and
// values of different sizes, chunks, a sink), in both engines, and of everything in the float32 engine.
//
// grouped_attention_kernel<T, JB>: block (token, key/value head and block of JB query heads of its group, split).  Keys
//   are visited in tiles of 64 aligned to absolute positions; split s of S takes the tiles whose index is s modulo S.
//   A tile's rows (and its values, unless the values are the keys' first columns) are staged in shared memory with
//   16-byte loads, rows padded to an odd number of words.  Scores: a thread takes one key, JB / 2 heads and half of the
//   row's words; the queries wait in shared memory as float32, a word's heads side by side, so that a thread fetches
//   its heads' numbers 16 bytes at a time.  Softmax: online, one warp per head in turn, 32-bit.  Weighted values: a
//   thread takes the words tid, tid + 256, .. of the value rows for all JB heads, whose weights it fetches 16 bytes at
//   a time.  The block writes unnormalised sums, its maximum and its sum of
//   weights; grouped_combine_kernel merges the splits in order, adds the sink's term to the denominator (and multiplies by
//   the sigmoid of a gate logit per output element, where the layer has such gates) and rounds
//   once.  What a query computes depends on its position, the split count and the cache only.
//
// q: [T, H, d] (float32, or the cache's type); cache: pages of keys [G, P, d] then values [G, P, dv], or (latent)
// [P, d] whose first dv columns are the values; masks as in attention_ref.cu.  d and dv are multiples of 16 bytes.
#include "common.cuh"
#include "mma.cuh"

namespace air {

// a score with a soft cap: cap * tanh(s / cap) where cap > 0, else the score itself
__device__ __forceinline__ float capped(float s, float cap) { return cap > 0.f ? cap * tanhf(s / cap) : s; }


constexpr int GA_KT = 64;                 // keys per tile

template <typename T> struct Words;       // how elements lie in 32-bit words, and how many words of a value row a
template <> struct Words<float> { static constexpr int per = 1, ni = 3; };             // thread takes (rows of up to
template <> struct Words<__nv_bfloat16> { static constexpr int per = 2, ni = 2; };     // 256 * ni words)

// n floats (2, 4, 8 or 16) from shared memory, the address aligned to min(16, 4 n) bytes
template <int N> __device__ __forceinline__ void load_floats(const float* p, float (&v)[N]) {
    if constexpr (N == 2) {
        const float2 t = *reinterpret_cast<const float2*>(p);
        v[0] = t.x; v[1] = t.y;
    } else {
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            const float4 t = *reinterpret_cast<const float4*>(p + 4 * i);
            v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
        }
    }
}

template <typename T, int JB>
__global__ void __launch_bounds__(256)
grouped_attention_kernel(const void* __restrict__ q_any, int q_f32, const T* __restrict__ cache,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ token_seq,
                         const int* __restrict__ positions, float* __restrict__ part, int H, int G, int d, int dv, int P,
                         int window, int mask_mode, float scale, float softcap, int latent, int splits) {
    constexpr int JT = JB / 2, PER = Words<T>::per, NI = Words<T>::ni;
    extern __shared__ __align__(16) float smem[];
    pdl_enter(TR_ATT_GROUPED);
    const int t = blockIdx.x, split = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int slot = token_seq[t];
    if (slot < 0) return;
    const int J = H / G, hbs = (J + JB - 1) / JB;
    const int g = blockIdx.y / hbs, j0 = (blockIdx.y % hbs) * JB, nj = min(JB, J - j0), head0 = g * J + j0;
    const int pos = positions[t];
    const int lo = window > 0 ? (mask_mode == 1 ? pos - pos % window : max(0, pos - window + 1)) : 0;
    const int* bt = block_table + (size_t)slot * max_blocks;
    const int kw = d / PER, vw = dv / PER;                 // words per row
    const int ksw = kw | 1, vsw = vw | 1;                  // ... as staged: odd, so that rows fall into different banks
    // The queries lie word by word, all heads of a word together: [kw][JB][PER] floats, so that a thread's heads are
    // one or a few 16-byte loads.  The scores and then the weights lie key by key: [2][64][JB] (two halves of the dot
    // products' range, added up by the softmax; the weights in the first half).
    float* qs = smem;
    float* S = qs + JB * d;
    float* corr = S + 2 * GA_KT * JB;                      // [JB], then the running maximum and sum
    float* mrun = corr + JB;
    float* lrun = mrun + JB;
    int* pages = reinterpret_cast<int*>(lrun + JB);        // [64]: the page of each of the tile's keys
    uint32_t* Kw = reinterpret_cast<uint32_t*>(pages + GA_KT);  // [64][ksw]
    uint32_t* Vw = latent ? Kw : Kw + GA_KT * ksw;          // [64][vsw]
    const int vstride = latent ? ksw : vsw;
    for (int i = tid; i < JB * d; i += 256) {
        const int j = i / d, e = i % d;
        float v = 0.f;
        if (j < nj) {
            const size_t at = ((size_t)t * H + head0 + j) * d + e;
            v = q_f32 ? ((const float*)q_any)[at] : to_float(((const T*)q_any)[at]);
        }
        qs[((e / PER) * JB + j) * PER + e % PER] = v;
    }
    if (tid < JB) { mrun[tid] = -INFINITY; lrun[tid] = 0.f; }
    float acc[JB][NI][PER];
#pragma unroll
    for (int j = 0; j < JB; ++j)
#pragma unroll
        for (int i = 0; i < NI; ++i)
#pragma unroll
            for (int e = 0; e < PER; ++e) acc[j][i][e] = 0.f;
    const size_t page_stride = latent ? (size_t)P * d : (size_t)G * P * (d + dv);
    const int kchunks = d * (int)sizeof(T) / 16, vchunks = dv * (int)sizeof(T) / 16;
    for (int kt = lo / GA_KT + split; kt * GA_KT <= pos; kt += splits) {
        const int key0 = kt * GA_KT;
        __syncthreads();                                   // the tile before this one has been used
        if (tid < GA_KT) {                                 // (looked up once, so that the loads below do not wait in turn)
            const int key = key0 + tid;
            pages[tid] = key >= lo && key <= pos ? bt[key / P] : -1;
        }
        __syncthreads();
#pragma unroll 4
        for (int c = tid; c < GA_KT * kchunks; c += 256) {
            const int r = c / kchunks, cc = c % kchunks;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (pages[r] >= 0) {
                const T* row = cache + (size_t)pages[r] * page_stride +
                               (latent ? (size_t)((key0 + r) % P) * d : ((size_t)g * P + (key0 + r) % P) * d);
                v = *reinterpret_cast<const uint4*>(row + cc * (16 / sizeof(T)));
            }
            uint32_t* dst = Kw + r * ksw + cc * 4;
            dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
        }
        if (!latent)
#pragma unroll 4
            for (int c = tid; c < GA_KT * vchunks; c += 256) {
                const int r = c / vchunks, cc = c % vchunks;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (pages[r] >= 0) {
                    const T* row = cache + (size_t)pages[r] * page_stride + (size_t)G * P * d +
                                   ((size_t)g * P + (key0 + r) % P) * dv;
                    v = *reinterpret_cast<const uint4*>(row + cc * (16 / sizeof(T)));
                }
                uint32_t* dst = Vw + r * vsw + cc * 4;
                dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
            }
        __syncthreads();
        {   // scores: key kk, heads gq * JT .., half of the row's words
            const int kk = tid & 63, gq = (tid >> 6) & 1, half = tid >> 7;
            float s[JT];
#pragma unroll
            for (int jt = 0; jt < JT; ++jt) s[jt] = 0.f;
            const uint32_t* krow = Kw + kk * ksw;
            const int w1 = (half + 1) * (kw / 2);
#pragma unroll 2
            for (int w = half * (kw / 2); w < w1; ++w) {
                const uint32_t word = krow[w];
                float qv[JT * PER];
                load_floats<JT * PER>(qs + (w * JB + gq * JT) * PER, qv);
                if (PER == 2) {
                    const __nv_bfloat162 k2 = *reinterpret_cast<const __nv_bfloat162*>(&word);
                    const float k0 = __low2float(k2), k1 = __high2float(k2);
#pragma unroll
                    for (int jt = 0; jt < JT; ++jt) s[jt] = fmaf(k1, qv[jt * PER + PER - 1], fmaf(k0, qv[jt * PER], s[jt]));
                } else {
                    const float k0 = __uint_as_float(word);
#pragma unroll
                    for (int jt = 0; jt < JT; ++jt) s[jt] = fmaf(k0, qv[jt], s[jt]);
                }
            }
#pragma unroll
            for (int jt = 0; jt < JT; ++jt) S[(half * GA_KT + kk) * JB + gq * JT + jt] = s[jt];
        }
        __syncthreads();
        for (int j = warp; j < JB; j += 8) {
            const bool seen0 = key0 + lane >= lo && key0 + lane <= pos, seen1 = key0 + lane + 32 >= lo && key0 + lane + 32 <= pos;
            const float s0 = seen0 ? capped((S[lane * JB + j] + S[(GA_KT + lane) * JB + j]) * scale, softcap) : -INFINITY;
            const float s1 = seen1 ? capped((S[(lane + 32) * JB + j] + S[(GA_KT + lane + 32) * JB + j]) * scale, softcap) : -INFINITY;
            const float m_old = mrun[j];
            const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
            float p0 = 0.f, p1 = 0.f, c = 1.f;
            if (m_new != -INFINITY) {
                p0 = expf(s0 - m_new);
                p1 = expf(s1 - m_new);
                c = expf(m_old - m_new);
            }
            const float sum = warp_sum(p0 + p1);
            S[lane * JB + j] = p0;
            S[(lane + 32) * JB + j] = p1;
            if (lane == 0) { lrun[j] = lrun[j] * c + sum; mrun[j] = m_new; corr[j] = c; }
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < JB; ++j) {
            const float c = corr[j];
#pragma unroll
            for (int i = 0; i < NI; ++i)
#pragma unroll
                for (int e = 0; e < PER; ++e) acc[j][i][e] *= c;
        }
        for (int kk = 0; kk < GA_KT; ++kk) {
            float pv[JB];
            load_floats<JB>(S + kk * JB, pv);
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int w = tid + 256 * i;
                if (w >= vw) continue;
                const uint32_t word = Vw[kk * vstride + w];
                if (PER == 2) {
                    const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&word);
                    const float v0 = __low2float(v2), v1 = __high2float(v2);
#pragma unroll
                    for (int j = 0; j < JB; ++j) {
                        acc[j][i][0] = fmaf(pv[j], v0, acc[j][i][0]);
                        acc[j][i][PER - 1] = fmaf(pv[j], v1, acc[j][i][PER - 1]);
                    }
                } else {
                    const float v0 = __uint_as_float(word);
#pragma unroll
                    for (int j = 0; j < JB; ++j) acc[j][i][0] = fmaf(pv[j], v0, acc[j][i][0]);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < JB; ++j) {
        if (j >= nj) continue;
        float* dst = part + (((size_t)t * H + head0 + j) * splits + split) * (dv + 2);
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int w = tid + 256 * i;
            if (w >= vw) continue;
#pragma unroll
            for (int e = 0; e < PER; ++e) dst[w * PER + e] = acc[j][i][e];
        }
        if (tid == 0) { dst[dv] = mrun[j]; dst[dv + 1] = lrun[j]; }
    }
}

// grouped_attention_tc_kernel: the same block for a bfloat16 cache with both products on the tensor cores (m16n8k16,
// 32-bit accumulators): the 16 query heads of the block are the rows of the instruction.  What the 32-bit kernel keeps in
// float32 stays 32-bit in effect: a float32 query is split into two bfloat16 numbers (q = hi + lo, the products q.k
// added in 32-bit), and so is every weight of the softmax before it meets the values; scores, maxima, sums and the
// weights themselves are float32.  Scores: warp w takes keys 8w .. 8w + 7 of the tile; weighted values: warp w takes
// the columns' eighth w; the values' fragments come transposed out of the staged rows (ldmatrix.trans).
constexpr int GT_MAX_NT = 16;      // 8-column tiles of the values per warp: dv up to 1024

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src, bool valid) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;             // 0: the 16 bytes are zero-filled, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void split_bf16(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

__global__ void __launch_bounds__(256)
grouped_attention_tc_kernel(const void* __restrict__ q_any, int q_f32, const __nv_bfloat16* __restrict__ cache,
                            const int* __restrict__ block_table, int max_blocks, const int* __restrict__ token_seq,
                            const int* __restrict__ positions, float* __restrict__ part, int H, int G, int d, int dv,
                            int P, int window, int mask_mode, float scale, float softcap, int latent, int splits, int stages) {
    constexpr int JB = 16, PLD = GA_KT + 8;
    extern __shared__ __align__(16) float smem[];
    pdl_enter(TR_ATT_GROUPED);
    const int t = blockIdx.x, split = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int slot = token_seq[t];
    if (slot < 0) return;
    const int J = H / G, hbs = (J + JB - 1) / JB;
    const int g = blockIdx.y / hbs, j0 = (blockIdx.y % hbs) * JB, nj = min(JB, J - j0), head0 = g * J + j0;
    const int pos = positions[t];
    const int lo = window > 0 ? (mask_mode == 1 ? pos - pos % window : max(0, pos - window + 1)) : 0;
    const int* bt = block_table + (size_t)slot * max_blocks;
    const int kld = d + 8, vld = latent ? kld : dv + 8;      // elements per staged row: 16 bytes of padding
    float* S = smem;                                          // [16][64] scores
    float* corr = S + JB * GA_KT;                             // [16], then the running maximum and sum
    float* mrun = corr + JB;
    float* lrun = mrun + JB;
    int* pages = reinterpret_cast<int*>(lrun + JB);           // [2][64]
    __nv_bfloat16* Qh = reinterpret_cast<__nv_bfloat16*>(pages + 2 * GA_KT);  // [16][kld] (and Ql behind it)
    __nv_bfloat16* Ql = Qh + JB * kld;
    __nv_bfloat16* Ph = Ql + JB * kld;                        // [16][72] weights, high and low halves
    __nv_bfloat16* Pl = Ph + JB * PLD;
    __nv_bfloat16* K0 = Pl + JB * PLD;                        // per stage: keys [64][kld], then values [64][vld]
    const int stage_elems = GA_KT * kld + (latent ? 0 : GA_KT * vld);
    for (int i = tid; i < JB * d; i += 256) {
        const int j = i / d, e = i % d;
        __nv_bfloat16 hi = __float2bfloat16_rn(0.f), lw = hi;
        if (j < nj) {
            const size_t at = ((size_t)t * H + head0 + j) * d + e;
            if (q_f32) split_bf16(((const float*)q_any)[at], hi, lw);
            else hi = ((const __nv_bfloat16*)q_any)[at];
        }
        Qh[j * kld + e] = hi;
        Ql[j * kld + e] = lw;
    }
    if (tid < JB) { mrun[tid] = -INFINITY; lrun[tid] = 0.f; }
    const int ntiles = (dv + 7) / 8, per_warp = (ntiles + 7) / 8;      // 8-column tiles of the values, and a warp's share
    const int nt0 = warp * per_warp;
    float acc[GT_MAX_NT][4];
#pragma unroll
    for (int n = 0; n < GT_MAX_NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
    const size_t page_stride = latent ? (size_t)P * d : (size_t)G * P * (d + dv);
    const int kchunks = d / 8, vchunks = dv / 8;
    const int gq = lane >> 2, tq = lane & 3;
    const uint32_t qh_addr = (uint32_t)__cvta_generic_to_shared(Qh), ql_addr = (uint32_t)__cvta_generic_to_shared(Ql);
    const uint32_t ph_addr = (uint32_t)__cvta_generic_to_shared(Ph), pl_addr = (uint32_t)__cvta_generic_to_shared(Pl);
    // ldmatrix.x4 of a 16 x 16 block of A (rows = heads): lane l gives the address of row l % 16, columns 8 (l / 16) ..
    const int a_row = lane & 15, a_col = (lane >> 4) * 8;
    // A tile's rows are brought by cp.async (16 bytes each, rows outside the mask zero-filled).  With two stages the
    // next tile of this block is on its way while this one is used.
    auto bring = [&](int key0, int buf) {
        __nv_bfloat16* Kt = K0 + (size_t)buf * stage_elems;
        __nv_bfloat16* Vt = Kt + GA_KT * kld;
        const int* pg = pages + buf * GA_KT;
        for (int c = tid; c < GA_KT * kchunks; c += 256) {
            const int r = c / kchunks, cc = c % kchunks, page = pg[r];
            const __nv_bfloat16* row = cache + (size_t)max(page, 0) * page_stride +
                                       (latent ? (size_t)((key0 + r) % P) * d : ((size_t)g * P + (key0 + r) % P) * d);
            cp_async16(Kt + r * kld + cc * 8, row + cc * 8, page >= 0);
        }
        if (!latent)
            for (int c = tid; c < GA_KT * vchunks; c += 256) {
                const int r = c / vchunks, cc = c % vchunks, page = pg[r];
                const __nv_bfloat16* row = cache + (size_t)max(page, 0) * page_stride + (size_t)G * P * d +
                                           ((size_t)g * P + (key0 + r) % P) * dv;
                cp_async16(Vt + r * vld + cc * 8, row + cc * 8, page >= 0);
            }
        cp_async_commit();
    };
    auto look_up = [&](int key0, int buf) {
        if (tid < GA_KT) {
            const int key = key0 + tid;
            pages[buf * GA_KT + tid] = key >= lo && key <= pos ? bt[key / P] : -1;
        }
    };
    const int kt_first = lo / GA_KT + split;
    if (stages == 2 && kt_first * GA_KT <= pos) {
        look_up(kt_first * GA_KT, 0);
        __syncthreads();
        bring(kt_first * GA_KT, 0);
    }
    int turn = 0;
    for (int kt = kt_first; kt * GA_KT <= pos; kt += splits, ++turn) {
        const int key0 = kt * GA_KT;
        const int buf = stages == 2 ? (turn & 1) : 0;
        if (stages == 2) {
            const int next = (kt + splits) * GA_KT;
            if (next <= pos) {
                look_up(next, buf ^ 1);
                __syncthreads();
                bring(next, buf ^ 1);
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
        } else {
            look_up(key0, 0);
            __syncthreads();
            bring(key0, 0);
            cp_async_wait<0>();
        }
        __syncthreads();                                   // this tile's rows have landed, everybody's copies
        const __nv_bfloat16* Kt = K0 + (size_t)buf * stage_elems;
        const uint32_t vt_addr = (uint32_t)__cvta_generic_to_shared(latent ? Kt : Kt + GA_KT * kld);
        {   // scores of the keys 8 warp .. 8 warp + 7
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const __nv_bfloat16* krow = Kt + (8 * warp + gq) * kld + 2 * tq;
            for (int kk = 0; kk < d; kk += 16) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + kk);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + kk + 8);
                uint32_t a[4];
                ldmatrix_x4(a, qh_addr + (a_row * kld + kk + a_col) * 2);
                mma_bf16_16816(c, a[0], a[1], a[2], a[3], b0, b1);
                if (q_f32) {
                    ldmatrix_x4(a, ql_addr + (a_row * kld + kk + a_col) * 2);
                    mma_bf16_16816(c, a[0], a[1], a[2], a[3], b0, b1);
                }
            }
            S[gq * GA_KT + 8 * warp + 2 * tq] = c[0];
            S[gq * GA_KT + 8 * warp + 2 * tq + 1] = c[1];
            S[(gq + 8) * GA_KT + 8 * warp + 2 * tq] = c[2];
            S[(gq + 8) * GA_KT + 8 * warp + 2 * tq + 1] = c[3];
        }
        __syncthreads();
        for (int j = warp; j < JB; j += 8) {
            const bool seen0 = key0 + lane >= lo && key0 + lane <= pos, seen1 = key0 + lane + 32 >= lo && key0 + lane + 32 <= pos;
            const float s0 = seen0 ? capped(S[j * GA_KT + lane] * scale, softcap) : -INFINITY;
            const float s1 = seen1 ? capped(S[j * GA_KT + lane + 32] * scale, softcap) : -INFINITY;
            const float m_old = mrun[j];
            const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
            float p0 = 0.f, p1 = 0.f, c = 1.f;
            if (m_new != -INFINITY) {
                p0 = expf(s0 - m_new);
                p1 = expf(s1 - m_new);
                c = expf(m_old - m_new);
            }
            const float sum = warp_sum(p0 + p1);
            split_bf16(p0, Ph[j * PLD + lane], Pl[j * PLD + lane]);
            split_bf16(p1, Ph[j * PLD + lane + 32], Pl[j * PLD + lane + 32]);
            if (lane == 0) { lrun[j] = lrun[j] * c + sum; mrun[j] = m_new; corr[j] = c; }
        }
        __syncthreads();
        {   // weighted values: the columns 8 nt0 .. of this warp
            const float c_lo = corr[gq], c_hi = corr[gq + 8];
#pragma unroll
            for (int n = 0; n < GT_MAX_NT; ++n) {
                acc[n][0] *= c_lo; acc[n][1] *= c_lo; acc[n][2] *= c_hi; acc[n][3] *= c_hi;
            }
#pragma unroll
            for (int ks = 0; ks < GA_KT / 16; ++ks) {
                uint32_t ah[4], al[4];
                ldmatrix_x4(ah, ph_addr + (a_row * PLD + ks * 16 + a_col) * 2);
                ldmatrix_x4(al, pl_addr + (a_row * PLD + ks * 16 + a_col) * 2);
                // the values' fragments, two column tiles at a time: lane l gives the address of key ks * 16 + (l / 8 % 2) * 8
                // + l % 8 at column 8 (tile + l / 16)
                const int v_key = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
                for (int n = 0; n < GT_MAX_NT; n += 2) {
                    if (n >= per_warp || nt0 + n >= ntiles) break;
                    const int col = 8 * (nt0 + n + (lane >> 4));
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vt_addr + (v_key * vld + min(col, vld - 8)) * 2);
                    mma_bf16_16816(acc[n], ah[0], ah[1], ah[2], ah[3], b[0], b[1]);
                    mma_bf16_16816(acc[n], al[0], al[1], al[2], al[3], b[0], b[1]);
                    if (n + 1 < per_warp && nt0 + n + 1 < ntiles) {
                        mma_bf16_16816(acc[n + 1], ah[0], ah[1], ah[2], ah[3], b[2], b[3]);
                        mma_bf16_16816(acc[n + 1], al[0], al[1], al[2], al[3], b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();                                   // the tile has been used: its stage may be refilled
    }
    __syncthreads();
#pragma unroll
    for (int n = 0; n < GT_MAX_NT; ++n) {
        if (n >= per_warp || nt0 + n >= ntiles) continue;
        const int col = 8 * (nt0 + n) + 2 * tq;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int j = gq + 8 * half;
            if (j >= nj) continue;
            float* dst = part + (((size_t)t * H + head0 + j) * splits + split) * (dv + 2);
            if (col < dv) dst[col] = acc[n][2 * half];
            if (col + 1 < dv) dst[col + 1] = acc[n][2 * half + 1];
        }
    }
    if (tid < nj) {
        float* dst = part + (((size_t)t * H + head0 + tid) * splits + split) * (dv + 2);
        dst[dv] = mrun[tid];
        dst[dv + 1] = lrun[tid];
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
grouped_combine_kernel(const float* __restrict__ part, const int* __restrict__ token_seq, const float* __restrict__ sink,
                       T* __restrict__ out, int H, int dv, int splits, const float* __restrict__ gate, int ldg) {
    pdl_enter(TR_ATT_GROUPED);
    const int t = blockIdx.x, h = blockIdx.y;
    if (token_seq[t] < 0) return;
    const float* p = part + ((size_t)t * H + h) * splits * (dv + 2);
    float m = sink ? sink[h] : -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, p[s * (dv + 2) + dv]);
    float total = sink ? expf(sink[h] - m) : 0.f;
    for (int s = 0; s < splits; ++s) {
        const float ms = p[s * (dv + 2) + dv];
        if (ms != -INFINITY) total += p[s * (dv + 2) + dv + 1] * expf(ms - m);
    }
    const float inv = 1.f / total;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = p[s * (dv + 2) + dv];
            if (ms != -INFINITY) o += p[s * (dv + 2) + c] * expf(ms - m);
        }
        // (a gate per output element: the logits' sigmoid multiplies as the row is written)
        const float g = gate ? 1.f / (1.f + expf(-gate[(size_t)t * ldg + h * dv + c])) : 1.f;
        out[((size_t)t * H + h) * dv + c] = from_float<T>(o * inv * g);
    }
}

template <typename T, int JB>
int launch_grouped(const void* q, int q_f32, const void* cache, const int* block_table, int max_blocks,
                   const int* token_seq, const int* positions, float* part, int T_, int H, int G, int d, int dv, int P,
                   int window, int mask_mode, float scale, float softcap, int latent, int splits, cudaStream_t stream) {
    constexpr int PER = Words<T>::per;
    const int ksw = (d / PER) | 1, vsw = (dv / PER) | 1;
    const size_t smem = sizeof(float) * ((size_t)JB * d + 2 * JB * GA_KT + 3 * JB + GA_KT) +
                        4 * (size_t)GA_KT * (ksw + (latent ? 0 : vsw));
    if (smem > 227 * 1024) return AIR_ERR_BAD_ARGUMENT;
    auto kernel = grouped_attention_kernel<T, JB>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int J = H / G;
    dim3 grid(T_, G * ((J + JB - 1) / JB), splits);
    return launch(kernel, grid, 256, smem, stream, q, q_f32, (const T*)cache, block_table, max_blocks, token_seq,
                  positions, part, H, G, d, dv, P, window, mask_mode, scale, softcap, latent, splits);
}

}  // namespace air

// part: float32 [T, H, splits, dv + 2] of scratch.
AIR_API int air_grouped_attention(const void* q, int q_f32, const void* cache, int dtype, const int* block_table,
                                  int max_blocks, const int* token_seq, const int* positions, float* part, void* out,
                                  int T, int H, int G, int d, int dv, int P, int window, float scale, int mask_mode,
                                  const float* sink, int latent, int splits, float softcap, const float* gate, int ldg,
                                  cudaStream_t stream) {
    if (T <= 0) return 0;
    const int bytes = dtype == AIR_F32 ? 4 : 2;
    if (d <= 0 || dv <= 0 || dv > (dtype == AIR_F32 ? 768 : 1024) || (d * bytes) % 16 || (dv * bytes) % 16 || H <= 0 || G <= 0 ||
        H % G || splits <= 0 || splits > 65535 || mask_mode < 0 || mask_mode > 1 || (latent && (dv > d || G != 1)))
        return AIR_ERR_BAD_ARGUMENT;
    const int J = H / G;
    int rc = 0;
    if (dtype == AIR_BF16 && d % 16 == 0 && dv % 8 == 0 && dv <= 128 * air::GT_MAX_NT / 2 * 1) {
        // both products on the tensor cores
        const int kld = d + 8, vld = dv + 8;
        const size_t stage = 2 * ((size_t)air::GA_KT * kld + (latent ? 0 : (size_t)air::GA_KT * vld));
        const size_t fixed = sizeof(float) * (16 * air::GA_KT + 3 * 16 + 2 * air::GA_KT) +
                             2 * ((size_t)2 * 16 * kld + 2 * 16 * (air::GA_KT + 8));
        const int stages = fixed + 2 * stage <= 227 * 1024 ? 2 : 1;
        const size_t smem = fixed + stages * stage;
        if (smem <= 227 * 1024) {
            auto kernel = air::grouped_attention_tc_kernel;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            dim3 grid(T, G * ((J + 15) / 16), splits);
            rc = air::launch(kernel, grid, 256, smem, stream, q, q_f32, (const __nv_bfloat16*)cache, block_table,
                             max_blocks, token_seq, positions, part, H, G, d, dv, P, window, mask_mode, scale, softcap, latent,
                             splits, stages);
            if (rc) return rc;
            return air::launch(air::grouped_combine_kernel<__nv_bfloat16>, dim3(T, H), 128, 0, stream, part, token_seq,
                               sink, (__nv_bfloat16*)out, H, dv, splits, gate, ldg);
        }
    }
    AIR_DISPATCH(dtype, TT, {
        if (J > 4)
            rc = air::launch_grouped<TT, 16>(q, q_f32, cache, block_table, max_blocks, token_seq, positions, part, T, H,
                                             G, d, dv, P, window, mask_mode, scale, softcap, latent, splits, stream);
        else
            rc = air::launch_grouped<TT, 4>(q, q_f32, cache, block_table, max_blocks, token_seq, positions, part, T, H,
                                            G, d, dv, P, window, mask_mode, scale, softcap, latent, splits, stream);
        if (rc) return rc;
        return air::launch(air::grouped_combine_kernel<TT>, dim3(T, H), 128, 0, stream, part, token_seq, sink, (TT*)out,
                           H, dv, splits, gate, ldg);
    });
    return 0;
}

AIR_API int air_trace_set_attention_grouped(unsigned long long* buffer) { return air::set_trace_here(buffer); }
