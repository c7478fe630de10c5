// Attention of a prompt portion as two matrix products around a softmax, for layers whose keys and values the tile
// kernels do not take (a latent row per token, keys and values of different sizes, chunks, a sink).  The portion's
// visible keys are gathered from the pages into one dense block, the library multiplies (scores = Q K^T in 32-bit
// accumulators and output, then weights times values), and the softmax between the two is this file's:
//
// gather_keys_kernel: keys lo .. lo + L of one request from its pages into dense blocks.  Paged keys and values: a
//   page holds the keys [G, P, dk] and then the values [G, P, dv]; out: K [G, Lp, dk], V [G, Lp, dv].  Latent rows: a
//   page is [P, dk]; out: K [1, Lp, dk] only (the values are its first columns).  Rows L .. Lp are zeroed.
//
// masked_softmax_kernel: S [G, n * J, Lp] float32 (row (t, j): token t of the portion, head g * J + j) -> weights of the
//   same shape in bfloat16.  Column c is the key at position lo + c; the query of token t stands at pos0 + t and sees
//   keys up to its own: all, the last `window`, or (mask_mode 1) those of its chunk of `window` positions.  weights =
//   exp(scale * s - m) / (sum + exp(sink_h - m)), the sink's term only where `sink` is given (with a soft cap the
//   score is cap * tanh(scale * s / cap)); 32-bit throughout,
//   rounded once at the end.  Columns that are not seen, and L .. Lp, become 0.
#include "common.cuh"

namespace air {

template <typename T>
__global__ void __launch_bounds__(128)
gather_keys_kernel(const T* __restrict__ cache, const int* __restrict__ block_table, int lo, int L, int Lp, int G,
                   int dk, int dv, int P, int latent, T* __restrict__ K, T* __restrict__ V) {
    pdl_enter(TR_GATHER_KEYS);
    const int c = blockIdx.x;
    if (c >= L) {
        for (int i = threadIdx.x; i < G * dk; i += blockDim.x) K[((size_t)(i / dk) * Lp + c) * dk + i % dk] = from_float<T>(0.f);
        if (V)
            for (int i = threadIdx.x; i < G * dv; i += blockDim.x)
                V[((size_t)(i / dv) * Lp + c) * dv + i % dv] = from_float<T>(0.f);
        return;
    }
    const int key = lo + c;
    const int page = block_table[key / P];
    const int place = key % P;
    if (latent) {
        const T* src = cache + ((size_t)page * P + place) * dk;
        for (int i = threadIdx.x; i < dk; i += blockDim.x) K[(size_t)c * dk + i] = src[i];
        return;
    }
    const T* base = cache + (size_t)page * G * P * (dk + dv);
    for (int i = threadIdx.x; i < G * dk; i += blockDim.x) {
        const int g = i / dk, e = i % dk;
        K[((size_t)g * Lp + c) * dk + e] = base[((size_t)g * P + place) * dk + e];
    }
    for (int i = threadIdx.x; i < G * dv; i += blockDim.x) {
        const int g = i / dv, e = i % dv;
        V[((size_t)g * Lp + c) * dv + e] = base[(size_t)G * P * dk + ((size_t)g * P + place) * dv + e];
    }
}

// a score with a soft cap: cap * tanh(s / cap) where cap > 0, else the score itself
__device__ __forceinline__ float soft_capped(float s, float cap) { return cap > 0.f ? cap * tanhf(s / cap) : s; }

__global__ void __launch_bounds__(256)
masked_softmax_kernel(const float* __restrict__ S, __nv_bfloat16* __restrict__ W, int n, int J, int L, int Lp, int lo,
                      int pos0, int window, int mask_mode, float scale, const float* __restrict__ sink, float softcap) {
    __shared__ float scratch[32];
    pdl_enter(TR_MASKED_SOFTMAX);
    const size_t r = blockIdx.x;
    const int g = (int)(r / ((size_t)n * J)), t = (int)((r % ((size_t)n * J)) / J), j = (int)(r % J);
    const int qpos = pos0 + t;
    const int first = window > 0 ? (mask_mode == 1 ? qpos - qpos % window : max(0, qpos - window + 1)) : 0;
    const int c0 = max(first - lo, 0), c1 = min(qpos - lo + 1, L);      // the row's visible columns
    const float* s = S + r * Lp;
    __nv_bfloat16* w = W + r * Lp;
    const float sk = sink ? sink[g * J + j] : -INFINITY;
    float m = sk;
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) m = fmaxf(m, soft_capped(s[c] * scale, softcap));
    m = warp_max(m);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
    __syncthreads();
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) m = fmaxf(m, scratch[i]);
    float sum = 0.f;
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) sum += expf(soft_capped(s[c] * scale, softcap) - m);
    sum = block_sum(sum, scratch);
    if (sink) sum += expf(sk - m);
    const float inv = 1.f / sum;
    for (int c = threadIdx.x; c < Lp; c += blockDim.x)
        w[c] = __float2bfloat16_rn(c >= c0 && c < c1 ? expf(soft_capped(s[c] * scale, softcap) - m) * inv : 0.f);
}

}  // namespace air

AIR_API int air_gather_keys(const void* cache, int dtype, const int* block_table, int lo, int L, int Lp, int G, int dk,
                            int dv, int P, int latent, void* K, void* V, cudaStream_t stream) {
    if (Lp <= 0) return 0;
    if (L > Lp || lo < 0 || G <= 0 || (latent && G != 1) || (!latent && !V)) return AIR_ERR_BAD_ARGUMENT;
    AIR_DISPATCH(dtype, TT, return air::launch(air::gather_keys_kernel<TT>, Lp, 128, 0, stream, (const TT*)cache,
                                               block_table, lo, L, Lp, G, dk, dv, P, latent, (TT*)K, (TT*)V));
    return 0;
}

AIR_API int air_masked_softmax(const float* S, void* W, int G, int n, int J, int L, int Lp, int lo, int pos0, int window,
                               int mask_mode, float scale, const float* sink, float softcap, cudaStream_t stream) {
    const long long rows = (long long)G * n * J;
    if (rows <= 0) return 0;
    if (rows > 2147483647LL || L > Lp) return AIR_ERR_BAD_ARGUMENT;
    return air::launch(air::masked_softmax_kernel, (unsigned)rows, 256, 0, stream, S, (__nv_bfloat16*)W, n, J, L, Lp, lo,
                       pos0, window, mask_mode, scale, sink, softcap);
}

AIR_API int air_trace_set_attention_gathered(unsigned long long* buffer) { return air::set_trace_here(buffer); }
