// Paged attention with 32-bit arithmetic for any batch: portions of prompts and single
// decoded tokens alike.  It is the kernel of the float32 path and the fallback of the
// bfloat16 path for head sizes that the tensor-core kernels do not take.
//
// One block per (token, query head), four warps.  Keys are visited in blocks of 32 aligned
// to their absolute position; warp w takes the blocks whose index is w modulo 4, keeps a
// running maximum, sum and weighted value (online softmax), and the four partial results
// are merged in a fixed order.  What a query computes therefore depends only on its
// position and on the cache's contents, not on how the tokens were cut into steps or on
// what else is in the batch.
//
// q: [T, H, d], out: [T, H, dv].  cache: a page holds the keys [K, P, d] and behind them the values [K, P, dv]
// (with dv == d that is [page, 2, K, P, d]).  block_table: [slots, max_blocks], row token_seq[t] for token t
// (negative: padding, skipped).
// A query at position p sees keys max(0, p - window + 1) .. p (window 0: all keys); with mask_mode 1 `window` is the
// size of a chunk instead, and the query sees the keys p - p % window .. p (those of its own chunk, counted from
// position 0 of the request).  With `sink` (float32 [H]) the softmax's denominator holds one more term exp(sink[h]):
// a bare logit that `scale` does not touch and that brings nothing to the output.  With `latent` a page is [P, d] (one row per token, no heads): every
// query head reads the same row as its key, and the row's first dv elements as its value.  q is float32 if q_f32,
// else of the cache's type.
// score = scale * q.k, and with softcap > 0 then softcap * tanh(score / softcap).  With `gate` [T, H] (float32) a
// head's output is multiplied by its token's gate.
#include "common.cuh"

namespace air {

constexpr int ATT_WARPS = 4;

template <typename T, int ATT_MAX_D>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_ref_kernel(const void* __restrict__ q_any, int q_f32, const T* __restrict__ cache,
                           const int* __restrict__ block_table, int max_blocks,
                           const int* __restrict__ token_seq, const int* __restrict__ positions,
                           T* __restrict__ out, const float* __restrict__ gate, int H, int K, int d, int dv, int P,
                           int window, float scale, float softcap, int mask_mode, const float* __restrict__ sink,
                           int latent) {
    __shared__ float sq[ATT_MAX_D];
    __shared__ float sm[ATT_WARPS], sl[ATT_WARPS];
    __shared__ float sacc[ATT_WARPS][ATT_MAX_D];
    pdl_enter(TR_ATT_REF);
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (token_seq[t] < 0) return;  // padding
    const int pos = positions[t];
    const int kvh = (int)(((long long)h * K) / H);
    const int* bt = block_table + (size_t)token_seq[t] * max_blocks;
    const int lo = window > 0 ? (mask_mode == 1 ? pos - pos % window : max(0, pos - window + 1)) : 0;

    if (q_f32)
        for (int i = threadIdx.x; i < d; i += blockDim.x) sq[i] = ((const float*)q_any)[((size_t)t * H + h) * d + i];
    else
        for (int i = threadIdx.x; i < d; i += blockDim.x) sq[i] = to_float(((const T*)q_any)[((size_t)t * H + h) * d + i]);
    __syncthreads();

    const int chunks = (dv + 31) / 32;
    float acc[ATT_MAX_D / 32];
#pragma unroll
    for (int c = 0; c < ATT_MAX_D / 32; ++c) acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;

    const size_t page_stride = latent ? (size_t)P * d : (size_t)K * P * (d + dv);
    const size_t v_offset = latent ? 0 : (size_t)K * P * d;
    const int v_stride = latent ? d : dv;
    for (int b = (lo / 32 / ATT_WARPS) * ATT_WARPS + warp; b * 32 <= pos; b += ATT_WARPS) {
        const int key = b * 32 + lane;
        const bool valid = key >= lo && key <= pos;
        size_t base = 0;      // of the key's value
        float s = -INFINITY;
        if (valid) {
            const int page = bt[key / P];
            const size_t place = (size_t)kvh * P + (size_t)(key % P);
            base = (size_t)page * page_stride + v_offset + place * v_stride;
            const T* kp = cache + (size_t)page * page_stride + place * d;
            float dot = 0.f;
            for (int i = 0; i < d; ++i) dot = fmaf(sq[i], to_float(kp[i]), dot);
            s = dot * scale;
            if (softcap > 0.f) s = softcap * tanhf(s / softcap);
        }
        const float bm = warp_max(s);
        if (bm == -INFINITY) continue;  // the whole block is outside the window
        const float m_new = fmaxf(m, bm);
        const float corr = expf(m - m_new);  // 0 when m was -inf
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int c = 0; c < ATT_MAX_D / 32; ++c) acc[c] *= corr;
        m = m_new;
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const unsigned long long bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
            if (pj == 0.f) continue;  // same for the whole warp
            const T* vp = cache + bj;
#pragma unroll
            for (int c = 0; c < ATT_MAX_D / 32; ++c) {
                const int i = c * 32 + lane;
                if (c < chunks && i < dv) acc[c] = fmaf(pj, to_float(vp[i]), acc[c]);
            }
        }
    }
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
    for (int c = 0; c < ATT_MAX_D / 32; ++c) {
        const int i = c * 32 + lane;
        if (c < chunks && i < dv) sacc[warp][i] = acc[c];
    }
    __syncthreads();
    float mm = sink ? sink[h] : -INFINITY;
    for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, sm[w]);
    float total = sink ? expf(sink[h] - mm) : 0.f;
    float weight[ATT_WARPS];
    for (int w = 0; w < ATT_WARPS; ++w) {
        weight[w] = sm[w] == -INFINITY ? 0.f : expf(sm[w] - mm);
        total += sl[w] * weight[w];
    }
    const float inv = (gate ? gate[(size_t)t * H + h] : 1.f) / total;
    for (int i = threadIdx.x; i < dv; i += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < ATT_WARPS; ++w) o += sacc[w][i] * weight[w];
        out[((size_t)t * H + h) * dv + i] = from_float<T>(o * inv);
    }
}

}  // namespace air

AIR_API int air_paged_attention_ref(const void* q, int q_f32, const void* cache, int dtype, const int* block_table,
                                    int max_blocks, const int* token_seq, const int* positions, void* out,
                                    const float* gate, int T, int H, int K, int d, int dv, int P, int window,
                                    float scale, float softcap, int mask_mode, const float* sink, int latent,
                                    cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || d > 640 || dv <= 0 || dv > 640 || H <= 0 || K <= 0 || H > 65535 || mask_mode < 0 || mask_mode > 1 ||
        (latent && (dv > d || K != 1)))
        return AIR_ERR_BAD_ARGUMENT;
    dim3 grid(T, H);
    AIR_DISPATCH(dtype, TT, {
        if (d <= 256 && dv <= 256)
            return air::launch(air::paged_attention_ref_kernel<TT, 256>, grid, air::ATT_WARPS * 32, 0, stream, q, q_f32,
                               (const TT*)cache, block_table, max_blocks, token_seq, positions, (TT*)out, gate, H, K,
                               d, dv, P, window, scale, softcap, mask_mode, sink, latent);
        return air::launch(air::paged_attention_ref_kernel<TT, 640>, grid, air::ATT_WARPS * 32, 0, stream, q, q_f32,
                           (const TT*)cache, block_table, max_blocks, token_seq, positions, (TT*)out, gate, H, K, d,
                           dv, P, window, scale, softcap, mask_mode, sink, latent);
    });
    return 0;
}

AIR_API int air_trace_set_attention_ref(unsigned long long* buffer) { return air::set_trace_here(buffer); }
