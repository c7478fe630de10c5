// What stands between the fused projection of an attention layer and its attention kernel, for layers whose
// keys and values differ in size or that want more than a bias and a rotation:
//
//   proj [T, ld] float32 holds, per token, q (H heads of dk), k (G heads of dk), v (G heads of dv) and, where the
//   layer gates its heads, H gate logits, in this order.  Per token: add the bias; rotate the first `rot` elements
//   of every head of q and k (element i with i + rot/2, angle position * inv_freq[i], evaluated here in 32-bit);
//   mix the values with those of an earlier layer, v = (1 - lambda) v + lambda v_first (v_mode 2), or hand them on
//   as v_first (v_mode 1); write q to q_out [T, H, dk], k and v into the token's place in the pages, and
//   sigmoid(gate logits) to gate_out [T, H].
//
// A page holds the keys [G, P, dk] and behind them the values [G, P, dv]; with dk == dv that is [2, G, P, d], the
// layout of the other attention kernels.
#include "common.cuh"

namespace air {

template <typename TO>
__global__ void __launch_bounds__(1024)
qkv_prepare_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias,
                   const float* __restrict__ inv_freq, int rot, const int* __restrict__ positions,
                   const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_blocks,
                   TO* __restrict__ q_out, TO* __restrict__ cache, float* __restrict__ gate_out,
                   float* __restrict__ v_first, int v_mode, const float* __restrict__ lambda,
                   int H, int G, int dk, int dv, int P, int* status) {
    pdl_enter(TR_QKV_PREPARE);
    const int t = blockIdx.x;
    const int slot = token_seq[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const float* in = proj + (size_t)t * ld;
    const int half = rot / 2;
    const int page = block_table[(size_t)slot * max_blocks + pos / P];
    TO* kdst = nullptr;
    TO* vdst = nullptr;
    if (page < 0) {
        if (threadIdx.x == 0 && status) atomicExch(status, 2);
    } else {
        TO* base = cache + (size_t)page * G * P * (dk + dv);
        kdst = base + (size_t)(pos % P) * dk;
        vdst = base + (size_t)G * P * dk + (size_t)(pos % P) * dv;
    }
    // q and k: one item per pair of rotated elements and per element behind the rotated part
    const int per_head = dk - half;
    for (int idx = threadIdx.x; idx < (H + G) * per_head; idx += blockDim.x) {
        const int head = idx / per_head, j = idx % per_head;
        const int col = head * dk;
        const int i0 = j < half ? j : j + half;
        float a = in[col + i0] + (bias ? bias[col + i0] : 0.f), b = 0.f;
        if (j < half) {
            b = in[col + i0 + half] + (bias ? bias[col + i0 + half] : 0.f);
            float s, c;
            sincosf((float)pos * inv_freq[j], &s, &c);
            const float ra = a * c - b * s, rb = b * c + a * s;
            a = ra;
            b = rb;
        }
        TO* dst = head < H ? q_out + ((size_t)t * H + head) * dk
                           : (kdst ? kdst + (size_t)(head - H) * P * dk : nullptr);
        if (dst) {
            dst[i0] = from_float<TO>(a);
            if (j < half) dst[i0 + half] = from_float<TO>(b);
        }
    }
    const int vcol = (H + G) * dk;
    const float lam = v_mode == 2 ? lambda[0] : 0.f;
    for (int idx = threadIdx.x; idx < G * dv; idx += blockDim.x) {
        float v = in[vcol + idx] + (bias ? bias[vcol + idx] : 0.f);
        if (v_mode == 1) v_first[(size_t)t * G * dv + idx] = v;
        else if (v_mode == 2) v = (1.f - lam) * v + lam * v_first[(size_t)t * G * dv + idx];
        if (vdst) vdst[(size_t)(idx / dv) * P * dv + idx % dv] = from_float<TO>(v);
    }
    if (gate_out) {
        const int gcol = vcol + G * dv;
        for (int h = threadIdx.x; h < H; h += blockDim.x) {
            const float z = in[gcol + h] + (bias ? bias[gcol + h] : 0.f);
            gate_out[(size_t)t * H + h] = 1.f / (1.f + expf(-z));
        }
    }
}

}  // namespace air

AIR_API int air_qkv_prepare(const float* proj, int ld, const float* bias, const float* inv_freq, int rot,
                            const int* positions, const int* token_seq, const int* block_table, int max_blocks,
                            void* q_out, void* cache, int out_dtype, float* gate_out, float* v_first, int v_mode,
                            const float* lambda, int T, int H, int G, int dk, int dv, int P, int* status,
                            cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > dk || (rot & 1) || (rot > 0 && !inv_freq) || v_mode < 0 || v_mode > 2 ||
        (v_mode && !v_first) || (v_mode == 2 && !lambda))
        return AIR_ERR_BAD_ARGUMENT;
    AIR_DISPATCH(out_dtype, TO, return air::launch(air::qkv_prepare_kernel<TO>, T, T <= 64 ? 1024 : 256, 0, stream, proj, ld, bias,
                                                   inv_freq, rot, positions, token_seq, block_table, max_blocks,
                                                   (TO*)q_out, (TO*)cache, gate_out, v_first, v_mode, lambda, H, G, dk,
                                                   dv, P, status));
    return 0;
}

AIR_API int air_trace_set_attention_prepare(unsigned long long* buffer) { return air::set_trace_here(buffer); }

// The same step for layers that normalise queries and keys per head before they rotate them, and whose rotation may
// pair neighbours:
//
//   q and k heads: x <- x / sqrt(mean(x^2) + eps) * w (w [dk], one for all heads of q, one for all heads of k; absent:
//   no norm); then the first `rot` elements are rotated, pair j by the angle position * freq[j], where pair j is
//   (2j, 2j + 1) (pairing 1) or (j, j + rot/2) (pairing 0); cos and sin are multiplied by `magnitude`.  The angle is
//   the product of the position and a 64-bit frequency, and its cos and sin are taken in 64-bit, once per token.
//   v is copied.  Pages as above.  A bias (float32 [(H + G) dk + G dv]) is added to q, k and v first.  With `whole`
//   the norm is taken over ALL heads of q at once (and all heads of k): x / sqrt(mean over H dk (x^2) + eps) * w with
//   w of that whole size (q_w [H dk], k_w [G dk]).
//
// One block per token, one warp per head of q or k; a lane holds up to QKN_PAIRS pairs of its head.
namespace air {

constexpr int QKN_PAIRS = 4;      // head sizes up to 64 * QKN_PAIRS

template <typename TO>
__global__ void __launch_bounds__(256)
qk_normed_prepare_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ q_w,
                         const float* __restrict__ k_w, float eps, const double* __restrict__ freq, int rot,
                         int pairing, float magnitude, const int* __restrict__ positions,
                         const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_blocks,
                         TO* __restrict__ q_out, TO* __restrict__ cache, int H, int G, int dk, int dv, int P,
                         int* status, const float* __restrict__ bias, int whole) {
    __shared__ float cs[128], sn[128], scratch[32];
    pdl_enter(TR_QK_NORMED_PREPARE);
    const int t = blockIdx.x;
    const int slot = token_seq[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const float* in = proj + (size_t)t * ld;
    const int half = rot / 2;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        double s, c;
        sincos((double)pos * freq[j], &s, &c);
        cs[j] = (float)c * magnitude;
        sn[j] = (float)s * magnitude;
    }
    const int page = block_table[(size_t)slot * max_blocks + pos / P];
    TO* kdst = nullptr;
    TO* vdst = nullptr;
    if (page < 0) {
        if (threadIdx.x == 0 && status) atomicExch(status, 2);
    } else {
        TO* base = cache + (size_t)page * G * P * (dk + dv);
        kdst = base + (size_t)(pos % P) * dk;
        vdst = base + (size_t)G * P * dk + (size_t)(pos % P) * dv;
    }
    __syncthreads();
    float whole_q = 1.f, whole_k = 1.f;
    if (whole && q_w) {      // one scale for all heads of q and one for all heads of k
        // (four loads of a thread under way at once: the sums are a chain of latencies otherwise)
        float sq = 0.f, sk = 0.f;
        const int n = (H + G) * dk, step = blockDim.x;
        for (int i0 = threadIdx.x; i0 < n; i0 += 4 * step) {
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * step;
                v[u] = i < n ? in[i] + (bias ? bias[i] : 0.f) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (i0 + u * step < H * dk) sq = fmaf(v[u], v[u], sq);
                else sk = fmaf(v[u], v[u], sk);
            }
        }
        whole_q = 1.f / sqrtf(block_sum(sq, scratch) / (float)(H * dk) + eps);
        whole_k = 1.f / sqrtf(block_sum(sk, scratch) / (float)(G * dk) + eps);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int pairs = dk / 2;
    for (int head = warp; head < H + G; head += warps) {
        const float* x = in + (size_t)head * dk;
        const float* hb = bias ? bias + (size_t)head * dk : nullptr;
        const float* w = head < H ? q_w : k_w;
        if (w && whole) w += (size_t)(head < H ? head : head - H) * dk;
        float a[QKN_PAIRS], b[QKN_PAIRS];
        int ia[QKN_PAIRS], ib[QKN_PAIRS];
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < QKN_PAIRS; ++c) {
            const int j = lane + 32 * c;
            a[c] = b[c] = 0.f;
            ia[c] = ib[c] = 0;
            if (j < pairs) {
                ia[c] = (pairing == 0 && j < half) ? j : 2 * j;
                ib[c] = (pairing == 0 && j < half) ? j + half : 2 * j + 1;
                a[c] = x[ia[c]] + (hb ? hb[ia[c]] : 0.f);
                b[c] = x[ib[c]] + (hb ? hb[ib[c]] : 0.f);
                ss += a[c] * a[c] + b[c] * b[c];
            }
        }
        ss = warp_sum(ss);
        const float scale = !w ? 1.f : whole ? (head < H ? whole_q : whole_k) : 1.f / sqrtf(ss / (float)dk + eps);
        TO* dst = head < H ? q_out + ((size_t)t * H + head) * dk
                           : (kdst ? kdst + (size_t)(head - H) * P * dk : nullptr);
#pragma unroll
        for (int c = 0; c < QKN_PAIRS; ++c) {
            const int j = lane + 32 * c;
            if (j >= pairs) continue;
            float u = a[c], v = b[c];
            if (w) {
                u = u * scale * w[ia[c]];
                v = v * scale * w[ib[c]];
            }
            if (j < half) {
                const float ru = u * cs[j] - v * sn[j], rv = v * cs[j] + u * sn[j];
                u = ru;
                v = rv;
            }
            if (dst) {
                dst[ia[c]] = from_float<TO>(u);
                dst[ib[c]] = from_float<TO>(v);
            }
        }
    }
    const int vcol = (H + G) * dk;
    if (vdst)
        for (int idx = threadIdx.x; idx < G * dv; idx += blockDim.x)
            vdst[(size_t)(idx / dv) * P * dv + idx % dv] =
                from_float<TO>(in[vcol + idx] + (bias ? bias[vcol + idx] : 0.f));
}

}  // namespace air

AIR_API int air_qk_normed_prepare(const float* proj, int ld, const float* q_w, const float* k_w, float eps,
                                  const double* freq, int rot, int pairing, float magnitude, const int* positions,
                                  const int* token_seq, const int* block_table, int max_blocks, void* q_out,
                                  void* cache, int out_dtype, int T, int H, int G, int dk, int dv, int P, int* status,
                                  const float* bias, int whole, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > dk || (rot & 1) || (dk & 1) || rot > 256 || dk > 64 * air::QKN_PAIRS || (rot > 0 && !freq) ||
        pairing < 0 || pairing > 1 || (!q_w) != (!k_w))
        return AIR_ERR_BAD_ARGUMENT;
    AIR_DISPATCH(out_dtype, TO, return air::launch(air::qk_normed_prepare_kernel<TO>, T, 256, 0, stream, proj, ld, q_w,
                                                   k_w, eps, freq, rot, pairing, magnitude, positions, token_seq,
                                                   block_table, max_blocks, (TO*)q_out, (TO*)cache, H, G, dk, dv, P,
                                                   status, bias, whole));
    return 0;
}
