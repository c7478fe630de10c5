// What stands between the first projection of a latent-attention layer and its attention kernel.
//
//   proj [T, ld] float32 holds, per token, q (H heads of [d plain | rot rotated]) and, where the layer makes its own
//   latent (owns), behind them the latent c (R columns) and one rotated key part kr (rot columns) for all heads.
//   Per token: c <- c / sqrt(mean(c^2) + eps) * w_c; kr and the rotated part of every head of q are turned, element i
//   with i + rot/2, by the angle position * freq[i] (a 64-bit product, cos and sin taken in 64-bit once per token);
//   the row [c | kr] goes to the token's place in the pages ([P, R + rot] per page, no heads); the plain part of q goes
//   to q_plain [T, H, d] (the matrix product that absorbs the key expansion reads it), the rotated part to
//   q_full[t, h, R : R + rot] (float32; that product fills q_full[t, h, 0 : R]).  rot may be 0 (no rotated parts).
//   Where the layer gates its heads, proj also holds one logit per head from column gate_col on, and
//   gate_out[t, h] = sigmoid(logit) (float32).
//
// One block per token.
#include "common.cuh"

namespace air {

template <typename TO>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ c_w, float eps,
                      const double* __restrict__ freq, const int* __restrict__ positions,
                      const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_blocks,
                      TO* __restrict__ q_plain, float* __restrict__ q_full, TO* __restrict__ cache, int owns, int H,
                      int d, int rot, int R, int P, float* __restrict__ gate_out, int gate_col, int* status, int vec) {
    __shared__ float cs[128], sn[128];
    __shared__ float scratch[32];
    pdl_enter(TR_LATENT_PREPARE);
    const int t = blockIdx.x;
    const int slot = token_seq[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const float* in = proj + (size_t)t * ld;
    const int half = rot / 2;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        double s, c;
        sincos((double)pos * freq[j], &s, &c);
        cs[j] = (float)c;
        sn[j] = (float)s;
    }
    __syncthreads();
    const int qw = d + rot;
    if (vec) {           // four numbers of a head at a time (d, rot and ld multiples of 4, 16-byte boundaries)
        for (int idx = threadIdx.x * 4; idx < H * d; idx += blockDim.x * 4) {
            const int h = idx / d, i = idx % d;
            float x[4];
            load4(in + h * qw + i, x);
            store4(q_plain + ((size_t)t * H + h) * d + i, x);
        }
    } else {
        for (int idx = threadIdx.x; idx < H * d; idx += blockDim.x) {
            const int h = idx / d, i = idx % d;
            q_plain[((size_t)t * H + h) * d + i] = from_float<TO>(in[h * qw + i]);
        }
    }
    for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
        const int h = idx / half, j = idx % half;
        const float u = in[h * qw + d + j], v = in[h * qw + d + j + half];
        float* dst = q_full + ((size_t)t * H + h) * (R + rot) + R;
        dst[j] = u * cs[j] - v * sn[j];
        dst[j + half] = v * cs[j] + u * sn[j];
    }
    if (gate_out)
        for (int h = threadIdx.x; h < H; h += blockDim.x)
            gate_out[(size_t)t * H + h] = 1.f / (1.f + expf(-in[gate_col + h]));
    if (!owns) return;
    const int page = block_table[(size_t)slot * max_blocks + pos / P];
    if (page < 0) {
        if (threadIdx.x == 0 && status) atomicExch(status, 2);
        return;
    }
    TO* row = cache + ((size_t)page * P + pos % P) * (R + rot);
    const float* c = in + (size_t)H * qw;
    float ss = 0.f;
    const bool vec_c = vec && R % 4 == 0;
    if (vec_c) {
        for (int i = threadIdx.x * 4; i < R; i += blockDim.x * 4) {
            float x[4];
            load4(c + i, x);
#pragma unroll
            for (int j = 0; j < 4; ++j) ss += x[j] * x[j];
        }
    } else {
        for (int i = threadIdx.x; i < R; i += blockDim.x) ss += c[i] * c[i];
    }
    const float total = block_sum(ss, scratch);
    const float scale = 1.f / sqrtf(total / (float)R + eps);
    if (vec_c) {
        for (int i = threadIdx.x * 4; i < R; i += blockDim.x * 4) {
            float x[4], wv[4];
            load4(c + i, x);
            load4(c_w + i, wv);
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] = x[j] * scale * wv[j];
            store4(row + i, x);
        }
    } else {
        for (int i = threadIdx.x; i < R; i += blockDim.x) row[i] = from_float<TO>(c[i] * scale * c_w[i]);
    }
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float u = c[R + j], v = c[R + j + half];
        row[R + j] = from_float<TO>(u * cs[j] - v * sn[j]);
        row[R + j + half] = from_float<TO>(v * cs[j] + u * sn[j]);
    }
}

}  // namespace air

AIR_API int air_latent_prepare(const float* proj, int ld, const float* c_w, float eps, const double* freq,
                               const int* positions, const int* token_seq, const int* block_table, int max_blocks,
                               void* q_plain, float* q_full, void* cache, int out_dtype, int owns, int T, int H, int d,
                               int rot, int R, int P, float* gate_out, int gate_col, int* status,
                               cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot < 0 || (rot & 1) || rot > 256 || (rot > 0 && !freq) || (owns && !c_w) || d <= 0 || R <= 0 ||
        (gate_out && (gate_col < H * (d + rot) + (owns ? R + rot : 0) || gate_col + H > ld)))
        return AIR_ERR_BAD_ARGUMENT;
    const int vec = d % 4 == 0 && rot % 4 == 0 && ld % 4 == 0 &&
                    (((uintptr_t)proj | (uintptr_t)c_w | (uintptr_t)q_plain | (uintptr_t)cache) & 15) == 0;
    AIR_DISPATCH(out_dtype, TO, return air::launch(air::latent_prepare_kernel<TO>, T, 256, 0, stream, proj, ld, c_w, eps,
                                                   freq, positions, token_seq, block_table, max_blocks, (TO*)q_plain,
                                                   q_full, (TO*)cache, owns, H, d, rot, R, P, gate_out, gate_col,
                                                   status, vec));
    return 0;
}

AIR_API int air_trace_set_latent_prepare(unsigned long long* buffer) { return air::set_trace_here(buffer); }
