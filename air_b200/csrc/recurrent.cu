// Mixers that carry a state of fixed size from token to token, over the step's flat batch: every entry of the
// batch brings the next tokens of one request (a portion of a prompt or one decoded token), rows
// q_start[e] .. q_start[e + 1] of the step, and slots[e] is the request's row of the state tensors (negative:
// padding, skipped).  Everything here is 32-bit: inputs, states and arithmetic.
//
//   short_conv_silu_kernel   y[t, c] = silu(sum_j w[c, j] x[t - (taps - 1 - j), c]): a causal convolution over time
//                            per channel whose last taps - 1 inputs are the state (zeros before a request's start);
//                            with act 0 the sum itself, without the SiLU
//   scan_prepare_kernel      what a scan reads per token (unit lengths, scales, decays), for all tokens side by side
//   linear_scan_kernel       a state S [d, dv] per head, updated token by token, read out after each update:
//                              DELTA  S = g S;  u = beta (v - S^T k);  S += k u^T;  o = S^T q   (one decay per head)
//                              GLA    S = diag(alpha) S + k v^T;  o = S^T q                      (a decay per key channel)
//                              HGRN   the same recurrence with k = 1 - alpha (the complement of the decay stands where
//                                     a key would); alpha = l + (1 - l) sigmoid(z + bias) with a lower bound l per
//                                     channel, q = silu(q)
//                              RET    S = g_h S + k v^T;  o = S^T q with one constant g_h per head (retention); q and k
//                                     are first rotated by the token's position, k then multiplied by a constant
//                            Columns of S do not depend on one another, so a block takes a few of them and a column is
//                            held in the registers of L lanes of one warp; the tokens of a portion are taken in order.
//                            What a token's output is depends on the state and the tokens before it only, not on how
//                            the request was cut into steps or on the rest of the batch.
//   gated_rmsnorm_kernel     out[t, h, :] = o / sqrt(mean(o^2) + eps) * w * silu(gate[t, h, :]) (without a gate: * w)
#include "common.cuh"

namespace air {

constexpr int CONV_MAX_TAPS = 16;
constexpr int CONV_THREADS = 128;

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// x [T, ld] (the first C columns), w [C, taps], state [slots, C, taps - 1] (oldest first), y [T, C].
// grid (channel blocks, entries, chunks of `chunk` tokens); the thread of a channel in the first chunk of an
// entry is the only one that reads or writes the channel's state.
__global__ void __launch_bounds__(CONV_THREADS)
short_conv_silu_kernel(const float* __restrict__ x, int ld, const float* __restrict__ w, float* __restrict__ state,
                       float* __restrict__ y, const int* __restrict__ q_start, const int* __restrict__ slots,
                       int C, int taps, int chunk, int act) {
    pdl_enter(TR_CONV);
    const int c = blockIdx.x * CONV_THREADS + threadIdx.x;
    const int e = blockIdx.y;
    const int slot = slots[e];
    if (c >= C || slot < 0) return;
    const int q0 = q_start[e], n = q_start[e + 1] - q0;
    const int t0 = blockIdx.z * chunk;
    if (t0 >= n && blockIdx.z > 0) return;
    const int t1 = min(n, t0 + chunk);
    const int keep = taps - 1;
    // Weights and window are held right-aligned in arrays of the largest size, so that every index is a
    // compile-time number (registers): wv[M - 1] is the current token's weight, win[j] the input M - 1 - j tokens
    // before the next one; the places in front of the taps hold zeros.
    constexpr int M = CONV_MAX_TAPS;
    const int lead = M - 1 - keep;            // unused places in front
    float wv[M], win[M - 1];
    float* st = state + ((size_t)slot * C + c) * keep;
#pragma unroll
    for (int j = 0; j < M; ++j) wv[j] = j >= lead ? w[(size_t)c * taps + (j - lead)] : 0.f;
#pragma unroll
    for (int j = 0; j < M - 1; ++j) {
        win[j] = 0.f;
        if (j >= lead) {
            const int idx = t0 - keep + (j - lead);      // the portion's token at this place, or (negative) the state's
            win[j] = idx >= 0 ? x[(size_t)(q0 + idx) * ld + c] : st[keep + idx];
        }
    }
    for (int t = t0; t < t1; ++t) {
        const float cur = x[(size_t)(q0 + t) * ld + c];
        float acc = wv[M - 1] * cur;
#pragma unroll
        for (int j = 0; j < M - 1; ++j)
            if (j >= lead) acc = fmaf(wv[j], win[j], acc);
        y[(size_t)(q0 + t) * C + c] = act ? silu_f(acc) : acc;
#pragma unroll
        for (int j = 0; j < M - 2; ++j) win[j] = win[j + 1];
        win[M - 2] = cur;
    }
    if (blockIdx.z == 0) {
        // The state after the portion: its last taps - 1 inputs.  A portion that this thread has taken whole leaves
        // them in the window (older ones from the state as it was included); a longer one has them all among its tokens
        // (a chunk is longer than the window).
#pragma unroll
        for (int j = 0; j < M - 1; ++j) {
            if (j >= lead) st[j - lead] = n <= chunk ? win[j] : x[(size_t)(q0 + n - keep + (j - lead)) * ld + c];
        }
    }
}

enum { SCAN_DELTA = 0, SCAN_GLA = 1, SCAN_HGRN = 2, SCAN_RET = 3 };
constexpr int SCAN_THREADS = 128;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem)
                 : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// What the scan reads per token, worked out for all tokens side by side (one block per token and head of q and k):
//   kq [T, G, 2, dpad]   k and then q of the head, as the recurrence takes them (unit length and q's scale for the
//                        delta rule, q's scale for gated linear attention), zeros from d to dpad
//   dec                  DELTA [T, H, 2]: g = exp(-exp(a_log) softplus(decay + dt_bias)) and b = sigmoid(beta)
//                        GLA   [T, H, dpad]: alpha = sigmoid(decay)^(1 / tau) per key channel, zeros from d on
//                        HGRN  [T, H, dpad]: alpha = l + (1 - l) sigmoid(decay + bias); kq's k is 1 - alpha (no k is
//                              read) and its q is silu(q) * q_scale
//                        RET   nothing: the decay is one constant per head, read by the scan from decay [H]; kq's q and
//                              k have their first `rot` elements rotated (element i with i + rot / 2, angle position *
//                              freq[i] as a 64-bit product, its cos and sin taken in 64-bit), q times q_scale, k times
//                              k_scale
struct ScanPrepArgs {
    const float* q; int ldq;         // [T, ldq]: head g's d elements at column g * d
    const float* k; int ldk;
    const float* decay; int ldd;     // DELTA: [T, ldd] one logit per head;  GLA: [T, ldd] d logits per head
    const float* beta; int ldb;      // DELTA: [T, ldb] one logit per head
    const float* a_log;              // DELTA: [H];  HGRN: the lower bounds l [H * d]
    const float* dt_bias;            // DELTA: [H];  HGRN: the gate's bias [H * d]
    const int* token_seq;
    float* kq;
    float* dec;
    int H, G, d, dpad;
    float q_scale, inv_tau, unit_eps;
    int unit;                        // q and k are divided by sqrt(sum of squares + unit_eps) first
    const int* positions;            // RET: [T]
    const double* freq;              // RET: [rot / 2]
    int rot;
    float k_scale;
};

template <int MODE>
__global__ void __launch_bounds__(128) scan_prepare_kernel(const ScanPrepArgs p) {
    __shared__ float scratch[32];
    pdl_enter(TR_SCAN);
    const int t = blockIdx.x, g = blockIdx.y;
    if (p.token_seq[t] < 0) return;
    const float* qin = p.q + (size_t)t * p.ldq + g * p.d;
    if (MODE == SCAN_HGRN) {
        const float* z = p.decay + (size_t)t * p.ldd + g * p.d;
        float* out = p.kq + ((size_t)t * p.G + g) * 2 * p.dpad;
        float* a = p.dec + ((size_t)t * p.H + g) * p.dpad;
        for (int r = threadIdx.x; r < p.dpad; r += blockDim.x) {
            float alpha = 0.f, k = 0.f, q = 0.f;
            if (r < p.d) {
                const float low = p.a_log[g * p.d + r];
                alpha = low + (1.f - low) / (1.f + expf(-(z[r] + p.dt_bias[g * p.d + r])));
                k = 1.f - alpha;
                q = silu_f(qin[r]) * p.q_scale;
            }
            a[r] = alpha;
            out[r] = k;
            out[p.dpad + r] = q;
        }
        return;
    }
    const float* kin = p.k + (size_t)t * p.ldk + g * p.d;
    if (MODE == SCAN_RET) {
        float* out = p.kq + ((size_t)t * p.G + g) * 2 * p.dpad;
        const int half = p.rot / 2;
        const double pos = (double)p.positions[t];
        for (int r = threadIdx.x; r < p.dpad; r += blockDim.x) {
            float k = 0.f, q = 0.f;
            if (r < p.d) {
                k = kin[r];
                q = qin[r];
                if (r < p.rot) {
                    const int j = r < half ? r : r - half;
                    double sn, cs;
                    sincos(pos * p.freq[j], &sn, &cs);
                    const float c = (float)cs, s = (float)sn;
                    const int other = r < half ? r + half : r - half;
                    // (a, b) -> (a c - b s, b c + a s): the first of a pair subtracts, the second adds
                    k = r < half ? k * c - kin[other] * s : k * c + kin[other] * s;
                    q = r < half ? q * c - qin[other] * s : q * c + qin[other] * s;
                }
            }
            out[r] = k * p.k_scale;
            out[p.dpad + r] = q * p.q_scale;
        }
        return;
    }
    float kf = 1.f, qf = p.q_scale;
    if (p.unit) {
        float sk = 0.f, sq = 0.f;
        for (int r = threadIdx.x; r < p.d; r += blockDim.x) {
            sk = fmaf(kin[r], kin[r], sk);
            sq = fmaf(qin[r], qin[r], sq);
        }
        kf = 1.f / sqrtf(block_sum(sk, scratch) + p.unit_eps);
        qf = p.q_scale / sqrtf(block_sum(sq, scratch) + p.unit_eps);
    }
    float* out = p.kq + ((size_t)t * p.G + g) * 2 * p.dpad;
    for (int r = threadIdx.x; r < p.dpad; r += blockDim.x) {
        out[r] = r < p.d ? kin[r] * kf : 0.f;
        out[p.dpad + r] = r < p.d ? qin[r] * qf : 0.f;
    }
    if (MODE == SCAN_GLA) {
        const float* z = p.decay + (size_t)t * p.ldd + g * p.d;
        float* a = p.dec + ((size_t)t * p.H + g) * p.dpad;
        for (int r = threadIdx.x; r < p.dpad; r += blockDim.x)
            a[r] = r < p.d ? expf(p.inv_tau * log_sigmoid_f(z[r])) : 0.f;
    } else if (g == 0) {
        for (int h = threadIdx.x; h < p.H; h += blockDim.x) {
            p.dec[((size_t)t * p.H + h) * 2] =
                expf(-expf(p.a_log[h]) * softplus_f(p.decay[(size_t)t * p.ldd + h] + p.dt_bias[h]));
            p.dec[((size_t)t * p.H + h) * 2 + 1] = 1.f / (1.f + expf(-p.beta[(size_t)t * p.ldb + h]));
        }
    }
}

struct ScanArgs {
    const float* kq;                 // [T, G, 2, dpad] (scan_prepare_kernel)
    const float* dec;                // DELTA [T, H, 2];  GLA [T, H, dpad]
    const float* v; int ldv;         // [T, ldv]: head h's dv elements at column h * dv
    float* state;                    // [slots, H, d, dv]
    float* out;                      // [T, H, dv]
    const int* q_start;
    const int* slots;
    int H, G, d, dv, L;              // G: heads of q and k (head h reads h / (H / G)); L lanes hold a column
    int tokens;                      // tokens staged in shared memory at a time (two such buffers)
};

// The staging is a copy (cp.async) into one of two buffers: the next tokens arrive while these are computed.
// A token's time is a chain of dependent instructions (decay, the sum over the column for the delta rule's
// prediction, the update), so the chain is kept short: L and R are compile-time (unrolled loops, no address
// arithmetic), and the read-out's sum over a column's lanes is not part of it: every lane leaves its partial sum
// in shared memory and the sums are taken, in a fixed order, when a buffer's tokens are written out.
template <int MODE, int R, int L>
__global__ void __launch_bounds__(SCAN_THREADS) linear_scan_kernel(const ScanArgs p) {
    extern __shared__ __align__(16) float smem[];
    pdl_enter(TR_SCAN);
    constexpr int cpw = 32 / L, CB = SCAN_THREADS / L, dpad = L * R;
    const int TK = p.tokens;
    const int e = blockIdx.z, h = blockIdx.y;
    const int slot = p.slots[e];
    if (slot < 0) return;
    const int q0 = p.q_start[e], n = p.q_start[e + 1] - q0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane / cpw;                                    // which rows of the column: l, l + L, l + 2L, ...
    const int cc = warp * cpw + lane % cpw;                      // column within the block
    const int col = blockIdx.x * CB + cc;
    const bool live = col < p.dv;
    const int g = h / (p.H / p.G);

    // a buffer: kq [TK][2][dpad], then (GLA) alpha [TK][dpad] or (DELTA) g, b [TK][2], then v [TK][CB]
    const int dec_floats = MODE == SCAN_GLA ? TK * dpad : (MODE == SCAN_RET ? 0 : ((2 * TK + 3) & ~3));
    const int buf_floats = TK * 2 * dpad + dec_floats + TK * CB;
    float* so = smem + 2 * buf_floats;                           // [TK][CB][L]: the lanes' partial read-outs

    auto stage = [&](int t0, int b) {
        const int cnt = min(TK, n - t0);
        float* bkq = smem + b * buf_floats;
        float* bdec = bkq + TK * 2 * dpad;
        float* bv = bdec + dec_floats;
        constexpr int per_token = 2 * dpad / 4;
        for (int idx = threadIdx.x; idx < cnt * per_token; idx += SCAN_THREADS) {
            const int tt = idx / per_token, c = idx % per_token;
            cp_async16(bkq + tt * 2 * dpad + 4 * c, p.kq + ((size_t)(q0 + t0 + tt) * p.G + g) * 2 * dpad + 4 * c);
        }
        if (MODE == SCAN_GLA) {
            constexpr int per = dpad / 4;
            for (int idx = threadIdx.x; idx < cnt * per; idx += SCAN_THREADS) {
                const int tt = idx / per, c = idx % per;
                cp_async16(bdec + tt * dpad + 4 * c, p.dec + ((size_t)(q0 + t0 + tt) * p.H + h) * dpad + 4 * c);
            }
        } else if (MODE == SCAN_DELTA) {
            for (int idx = threadIdx.x; idx < cnt * 2; idx += SCAN_THREADS)
                cp_async4(bdec + idx, p.dec + ((size_t)(q0 + t0 + idx / 2) * p.H + h) * 2 + (idx & 1));
        }
        for (int idx = threadIdx.x; idx < cnt * CB; idx += SCAN_THREADS) {
            const int tt = idx / CB, c = blockIdx.x * CB + idx % CB;
            if (c < p.dv) cp_async4(bv + idx, p.v + (size_t)(q0 + t0 + tt) * p.ldv + h * p.dv + c);
        }
        cp_async_commit();
    };

    stage(0, 0);
    const float ghead = MODE == SCAN_RET ? p.dec[h] : 0.f;      // the head's constant decay
    float S[R];
    float* st = p.state + ((size_t)slot * p.H + h) * p.d * p.dv;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = i * L + l;
        S[i] = (live && r < p.d) ? st[(size_t)r * p.dv + col] : 0.f;
    }

    int b = 0;
    for (int t0 = 0; t0 < n; t0 += TK, b ^= 1) {
        const int cnt = min(TK, n - t0);
        cp_async_wait_all();
        __syncthreads();                       // this buffer has landed; the other one and `so` are free again
        if (t0 + TK < n) stage(t0 + TK, b ^ 1);
        const float* bkq = smem + b * buf_floats;
        const float* bdec = bkq + TK * 2 * dpad;
        const float* bv = bdec + dec_floats;
        for (int tt = 0; tt < cnt; ++tt) {
            const float* kk = bkq + tt * 2 * dpad + l;
            const float* qq = kk + dpad;
            const float vv = live ? bv[tt * CB + cc] : 0.f;
            // (four partial sums each: the chain of dependent additions is a quarter as long)
            float orr[4] = {0.f, 0.f, 0.f, 0.f};
            if (MODE == SCAN_DELTA) {
                const float gv = bdec[2 * tt], bb = bdec[2 * tt + 1];
                float kr[R], pr[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    kr[i] = kk[i * L];
                    S[i] *= gv;
                    pr[i & 3] = fmaf(S[i], kr[i], pr[i & 3]);
                }
                float pred = (pr[0] + pr[1]) + (pr[2] + pr[3]);
#pragma unroll
                for (int off = 16; off >= cpw; off >>= 1) pred += __shfl_xor_sync(0xffffffffu, pred, off);
                const float u = bb * (vv - pred);
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    S[i] = fmaf(kr[i], u, S[i]);
                    orr[i & 3] = fmaf(S[i], qq[i * L], orr[i & 3]);
                }
            } else if (MODE == SCAN_RET) {
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    S[i] = fmaf(ghead, S[i], kk[i * L] * vv);
                    orr[i & 3] = fmaf(S[i], qq[i * L], orr[i & 3]);
                }
            } else {
                const float* aa = bdec + tt * dpad + l;
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    S[i] = fmaf(aa[i * L], S[i], kk[i * L] * vv);
                    orr[i & 3] = fmaf(S[i], qq[i * L], orr[i & 3]);
                }
            }
            so[(tt * CB + cc) * L + l] = (orr[0] + orr[1]) + (orr[2] + orr[3]);
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < cnt * CB; idx += SCAN_THREADS) {
            const int tt = idx / CB, c = blockIdx.x * CB + idx % CB;
            float o = 0.f;
#pragma unroll
            for (int j = 0; j < L; ++j) o += so[idx * L + j];
            if (c < p.dv) p.out[((size_t)(q0 + t0 + tt) * p.H + h) * p.dv + c] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = i * L + l;
        if (live && r < p.d) st[(size_t)r * p.dv + col] = S[i];
    }
}

// o [T, H, dv] float32; gate [T, ldg] float32 (head h at column h * dv) or null (no gate); w [dv]; out [T, H * dv].
// One warp per (token, head).
template <typename TO>
__global__ void __launch_bounds__(128)
gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ gate, int ldg, const float* __restrict__ w,
                     TO* __restrict__ out, const int* __restrict__ token_seq, int T, int H, int dv, float eps, int vec) {
    pdl_enter(TR_GATED);
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= T * H) return;
    const int t = item / H, h = item % H;
    if (token_seq[t] < 0) return;
    const float* row = o + (size_t)item * dv;
    float ss = 0.f;
    if (vec) {           // four columns per lane and access (dv and ldg multiples of 4, the tensors on 16-byte boundaries)
        for (int i = lane * 4; i < dv; i += 128) {
            float x[4];
            load4(row + i, x);
#pragma unroll
            for (int j = 0; j < 4; ++j) ss = fmaf(x[j], x[j], ss);
        }
        ss = warp_sum(ss);
        const float scale = rsqrtf(ss / (float)dv + eps);
        const float* gr = gate ? gate + (size_t)t * ldg + h * dv : nullptr;
        for (int i = lane * 4; i < dv; i += 128) {
            float x[4], wv[4], g[4];
            load4(row + i, x);
            load4(w + i, wv);
            if (gr) load4(gr + i, g);
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] = x[j] * scale * wv[j] * (gr ? silu_f(g[j]) : 1.f);
            store4(out + (size_t)item * dv + i, x);
        }
        return;
    }
    for (int i = lane; i < dv; i += 32) ss = fmaf(row[i], row[i], ss);
    ss = warp_sum(ss);
    const float scale = rsqrtf(ss / (float)dv + eps);
    const float* gr = gate ? gate + (size_t)t * ldg + h * dv : nullptr;
    for (int i = lane; i < dv; i += 32)
        out[(size_t)item * dv + i] = from_float<TO>(row[i] * scale * w[i] * (gr ? silu_f(gr[i]) : 1.f));
}

// rows of a column per lane: 16 up to 512 key channels, 32 beyond
static int scan_rows(int d) { return d <= 512 ? 16 : 32; }

// PREP: what scan_prepare_kernel works out; MODE: the recurrence (HGRN's is GLA's)
template <int PREP, int MODE = (PREP == SCAN_HGRN ? SCAN_GLA : PREP)>
static int launch_scan(const ScanPrepArgs& prep, const ScanArgs& a, int T, int S, cudaStream_t stream) {
    const int R = scan_rows(a.d), L = a.L, dpad = L * R;
    if (L < 1 || L > 32 || (L & (L - 1)) || dpad < a.d || prep.dpad != dpad || (R == 32 && L != 32))
        return AIR_ERR_BAD_ARGUMENT;
    if (a.H > 65535 || S > 65535 || prep.G > 65535) return AIR_ERR_BAD_ARGUMENT;
    int rc = launch(scan_prepare_kernel<PREP>, dim3(T, prep.G), 128, 0, stream, prep);
    if (rc) return rc;
    ScanArgs p = a;
    const int CB = SCAN_THREADS / L;
    // two buffers of `tokens` tokens each, and their partial read-outs, within 96 KB
    auto bytes = [&](int tk) {
        const size_t dec = MODE == SCAN_GLA ? (size_t)tk * dpad : (MODE == SCAN_RET ? 0 : (size_t)((2 * tk + 3) & ~3));
        return sizeof(float) * (2 * ((size_t)tk * 2 * dpad + dec + (size_t)tk * CB) + (size_t)tk * SCAN_THREADS);
    };
    int tk = 16;
    while (tk > 1 && bytes(tk) > 96 * 1024) tk /= 2;
    p.tokens = tk;
    size_t smem = bytes(tk);
    const dim3 grid((a.dv + CB - 1) / CB, a.H, S);
    // A block's time is the length of its chain, and blocks that share an SM's schedulers stretch one another's.
    // Measured (2,048 tokens, 128 blocks): 576 us when every block has an SM, 1,235 us when the blocks, launched
    // while the kernel before them was still leaving the SMs, had landed several to an SM.  So the kernel starts
    // only when its predecessor has ended (no programmatic launch), and while there are no more blocks than SMs (or
    // than twice the SMs) a block asks for so much shared memory that only one (two) of them fit an SM.
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long blocks = (long long)grid.x * grid.y * grid.z;
    if (blocks <= sms && smem < 120 * 1024) smem = 120 * 1024;
    else if (blocks <= 2ll * sms && smem < 80 * 1024) smem = 80 * 1024;
    auto go = [&](auto kernel) {
        if (smem > 48 * 1024) {
            cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (err != cudaSuccess) return (int)err;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(SCAN_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        return (int)cudaLaunchKernelEx(&cfg, kernel, p);
    };
    if (R == 32) return go(linear_scan_kernel<MODE, 32, 32>);
    switch (L) {
        case 1: return go(linear_scan_kernel<MODE, 16, 1>);
        case 2: return go(linear_scan_kernel<MODE, 16, 2>);
        case 4: return go(linear_scan_kernel<MODE, 16, 4>);
        case 8: return go(linear_scan_kernel<MODE, 16, 8>);
        case 16: return go(linear_scan_kernel<MODE, 16, 16>);
        default: return go(linear_scan_kernel<MODE, 16, 32>);
    }
}

}  // namespace air

AIR_API int air_short_conv_silu(const float* x, int ld, const float* w, float* state, float* y, const int* q_start,
                                const int* slots, int S, int C, int taps, int max_tokens, int act,
                                cudaStream_t stream) {
    if (S <= 0 || C <= 0) return 0;
    if (taps < 1 || taps > air::CONV_MAX_TAPS || S > 65535) return AIR_ERR_BAD_ARGUMENT;
    const int chunk = 64;
    int chunks = (max_tokens + chunk - 1) / chunk;
    if (chunks < 1) chunks = 1;
    if (chunks > 65535) return AIR_ERR_BAD_ARGUMENT;
    dim3 grid((C + air::CONV_THREADS - 1) / air::CONV_THREADS, S, chunks);
    return air::launch(air::short_conv_silu_kernel, grid, air::CONV_THREADS, 0, stream, x, ld, w, state, y, q_start,
                       slots, C, taps, chunk, act);
}

// kq: float32 workspace [T, G, 2, L * R] and dec: [T, H, 2] (mode 0) or [T, H, L * R] (modes 1, 2), with R = 16 up to
// 512 key channels and 32 beyond, L the power of two with L * R >= d.  Mode 3 (retention): decay is [H], the heads'
// constants, and no dec is needed; positions [T], freq float64 [rot / 2], k_scale as ScanPrepArgs says.
AIR_API int air_linear_scan(int mode, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                            const float* decay, int ldd, const float* beta, int ldb, const float* a_log,
                            const float* dt_bias, float* state, float* out, const int* q_start, const int* slots,
                            const int* token_seq, float* kq, float* dec, int T, int S, int H, int G, int d, int dv,
                            int L, float q_scale, float inv_tau, int unit, float unit_eps, const int* positions,
                            const double* freq, int rot, float k_scale, cudaStream_t stream) {
    if (S <= 0 || T <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || !kq || ((uintptr_t)kq & 15) ||
        (mode != air::SCAN_RET && (!dec || ((uintptr_t)dec & 15))))
        return AIR_ERR_BAD_ARGUMENT;
    air::ScanPrepArgs pr;
    pr.q = q; pr.ldq = ldq; pr.k = k; pr.ldk = ldk; pr.decay = decay; pr.ldd = ldd; pr.beta = beta; pr.ldb = ldb;
    pr.a_log = a_log; pr.dt_bias = dt_bias; pr.token_seq = token_seq; pr.kq = kq; pr.dec = dec; pr.H = H; pr.G = G;
    pr.d = d; pr.dpad = L * air::scan_rows(d); pr.q_scale = q_scale; pr.inv_tau = inv_tau; pr.unit_eps = unit_eps;
    pr.unit = unit; pr.positions = positions; pr.freq = freq; pr.rot = rot; pr.k_scale = k_scale;
    air::ScanArgs a;
    a.kq = kq; a.dec = dec; a.v = v; a.ldv = ldv; a.state = state; a.out = out; a.q_start = q_start; a.slots = slots;
    a.H = H; a.G = G; a.d = d; a.dv = dv; a.L = L; a.tokens = 0;
    if (mode == air::SCAN_DELTA) return air::launch_scan<air::SCAN_DELTA>(pr, a, T, S, stream);
    if (mode == air::SCAN_GLA) return air::launch_scan<air::SCAN_GLA>(pr, a, T, S, stream);
    if (mode == air::SCAN_HGRN) {
        if (G != H || !a_log || !dt_bias) return AIR_ERR_BAD_ARGUMENT;
        return air::launch_scan<air::SCAN_HGRN>(pr, a, T, S, stream);
    }
    if (mode == air::SCAN_RET) {
        if (G != H || !decay || rot < 0 || rot > d || (rot & 1) || (rot && (!positions || !freq)))
            return AIR_ERR_BAD_ARGUMENT;
        a.dec = decay;
        return air::launch_scan<air::SCAN_RET>(pr, a, T, S, stream);
    }
    return AIR_ERR_BAD_ARGUMENT;
}

AIR_API int air_gated_rmsnorm(const float* o, const float* gate, int ldg, const float* w, void* out, int out_dtype,
                              const int* token_seq, int T, int H, int dv, float eps, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int blocks = (T * H + 3) / 4;
    const int vec = dv % 4 == 0 && (!gate || ldg % 4 == 0) &&
                    (((uintptr_t)o | (uintptr_t)gate | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    AIR_DISPATCH(out_dtype, TO, return air::launch(air::gated_rmsnorm_kernel<TO>, blocks, 128, 0, stream, o, gate, ldg, w,
                                                   (TO*)out, token_seq, T, H, dv, eps, vec));
    return 0;
}

AIR_API int air_trace_set_recurrent(unsigned long long* buffer) { return air::set_trace_here(buffer); }
