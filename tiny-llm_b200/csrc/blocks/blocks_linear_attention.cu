// Linear attention with a per-channel decay (a recurrent mixer) over ragged batches, its state kept in fp32 slots.
//
// Per sequence and head a matrix S [dk, dv] is carried from token to token:
//     S <- diag(alpha_t) S + k_t v_t^T,      o_t = S^T (q_scale * q_t),
//     alpha_t = sigmoid(z_t + bias)^(1 / tau) = exp(log_sigmoid(z_t + bias) / tau)        (per key channel)
// The columns of S never mix, so a CTA owns 32 of them for one (sequence, head) and walks the sequence's new tokens in
// order; 4 lanes share a column, each holding every 4th row of it in registers.  The tokens' q, k and decays are staged
// 16 at a time in shared memory as fp32 (the decay is computed there, in fp32, from the fp32 logits).  A sequence that
// starts at position 0 starts from zero, whatever its slot held; otherwise the slot is read, and in both cases written
// back after the last token.  The order of every sum is fixed by the token and channel indices alone, so the result
// does not depend on how the tokens were cut into steps or on the rest of the batch.
#include "blocks_common.cuh"

namespace tlb {

constexpr int kLaCols = 32;    // state columns per CTA
constexpr int kLaLanes = 4;    // lanes per column
constexpr int kLaTokens = 16;  // tokens staged at a time

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename T, int KR /* rows per lane: dk <= 4 * KR */>
__global__ void __launch_bounds__(kLaCols * kLaLanes)
decay_scan_kernel(const T *__restrict__ q, long long q_token, long long q_head, const T *__restrict__ k, long long k_token, long long k_head,
                  const T *__restrict__ v, long long v_token, long long v_head, const float *__restrict__ z, long long z_token,
                  const T *__restrict__ z_bias, float inv_tau, float q_scale, int heads, int dk, int dv, const int32_t *__restrict__ seq_info,
                  float *__restrict__ state, long long slot_stride, int num_slots, float *__restrict__ out) {
    __shared__ float sq[kLaTokens * 4 * KR], sk[kLaTokens * 4 * KR], sa[kLaTokens * 4 * KR];
    __shared__ float sv[kLaTokens * kLaCols];
    const int s = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * kLaCols;
    const int first = seq_info[s * 4 + 0], count = seq_info[s * 4 + 1], start = seq_info[s * 4 + 2], slot = seq_info[s * 4 + 3];
    const int c = threadIdx.x / kLaLanes, r = threadIdx.x % kLaLanes;
    const int col = col0 + c;
    const bool col_ok = col < dv;
    const bool slot_ok = slot >= 0 && slot < num_slots;
    float *mine = state + (size_t)(slot_ok ? slot : 0) * slot_stride + (size_t)head * dk * dv;

    float S[KR];
#pragma unroll
    for (int i = 0; i < KR; ++i) {
        int row = r + kLaLanes * i;
        S[i] = (start > 0 && slot_ok && col_ok && row < dk) ? mine[(size_t)row * dv + col] : 0.f;
    }
    for (int t0 = 0; t0 < count; t0 += kLaTokens) {
        const int n = min(kLaTokens, count - t0);
        __syncthreads();
        for (int e = threadIdx.x; e < n * dk; e += blockDim.x) {
            int j = e / dk, d = e - j * dk;
            size_t tok = (size_t)(first + t0 + j);
            sq[j * 4 * KR + d] = to_f(q[tok * q_token + (size_t)head * q_head + d]) * q_scale;
            sk[j * 4 * KR + d] = to_f(k[tok * k_token + (size_t)head * k_head + d]);
            float logit = z[tok * z_token + (size_t)head * dk + d] + (z_bias ? to_f(z_bias[(size_t)head * dk + d]) : 0.f);
            sa[j * 4 * KR + d] = expf(log_sigmoid(logit) * inv_tau);
        }
        for (int e = threadIdx.x; e < n * kLaCols; e += blockDim.x) {
            int j = e / kLaCols, d = e - j * kLaCols;
            sv[e] = col0 + d < dv ? to_f(v[(size_t)(first + t0 + j) * v_token + (size_t)head * v_head + col0 + d]) : 0.f;
        }
        __syncthreads();
        for (int j = 0; j < n; ++j) {
            const float vj = sv[j * kLaCols + c];
            const float *qa = sq + j * 4 * KR, *ka = sk + j * 4 * KR, *aa = sa + j * 4 * KR;
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < KR; ++i) {
                int row = r + kLaLanes * i;
                if (row < dk) {
                    S[i] = fmaf(aa[row], S[i], ka[row] * vj);
                    o = fmaf(qa[row], S[i], o);
                }
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (r == 0 && col_ok) out[((size_t)(first + t0 + j) * heads + head) * dv + col] = o;
        }
    }
    if (slot_ok && col_ok) {
#pragma unroll
        for (int i = 0; i < KR; ++i) {
            int row = r + kLaLanes * i;
            if (row < dk) mine[(size_t)row * dv + col] = S[i];
        }
    }
}

// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * act(gate[t, h, :]); one warp per (token, head).  act 0 = none, 1 = silu.
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float *__restrict__ o, const T *__restrict__ w, float eps, const T *__restrict__ gate, long long g_token, int act,
                      T *__restrict__ out, long long rows, int heads, int dv) {
    long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const long long t = row / heads;
    const int head = (int)(row - t * heads);
    const float *src = o + (size_t)row * dv;
    float ss = 0.f;
    for (int d = lane; d < dv; d += 32) ss += src[d] * src[d];
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int d = lane; d < dv; d += 32) {
        float y = src[d] * inv * to_f(w[d]);
        if (gate) {
            float gv = to_f(gate[(size_t)t * g_token + (size_t)head * dv + d]);
            y *= act == 1 ? gv / (1.0f + expf(-gv)) : gv;
        }
        out[(size_t)row * dv + d] = from_f<T>(y);
    }
}

}  // namespace tlb

using namespace tlb;

extern "C" {

int tlb_decay_scan(const void *q, long long q_token, long long q_head, const void *k, long long k_token, long long k_head, const void *v,
                   long long v_token, long long v_head, const float *z, long long z_token, const void *z_bias, float tau, float q_scale, int heads,
                   int dk, int dv, const int32_t *seq_info, int num_seqs, float *state, long long slot_stride, int num_slots, float *out, int dtype,
                   void *stream) {
    if (num_seqs <= 0) return TL_OK;
    if (!q || !k || !v || !z || !seq_info || !state || !out || heads <= 0 || dk <= 0 || dv <= 0 || !(tau > 0.f) || num_slots <= 0)
        return tl::fail(TL_EINVAL, "decay_scan: bad argument");
    if (dk > 128) return tl::fail(TL_EINVAL, "decay_scan: key size %d > 128", dk);
    dim3 grid(num_seqs, heads, ceil_div(dv, kLaCols));
    cudaStream_t st = as_stream(stream);
    int kr = ceil_div(dk, kLaLanes);
#define TLB_DS(KRV)                                                                                                                               \
    decay_scan_kernel<T, KRV><<<grid, kLaCols * kLaLanes, 0, st>>>((const T *)q, q_token, q_head, (const T *)k, k_token, k_head, (const T *)v, v_token, \
                                                                  v_head, z, z_token, (const T *)z_bias, 1.0f / tau, q_scale, heads, dk, dv, seq_info, \
                                                                  state, slot_stride, num_slots, out)
    TLB_DISPATCH(dtype, "decay_scan", if (kr <= 8) TLB_DS(8); else if (kr <= 16) TLB_DS(16); else TLB_DS(32));
#undef TLB_DS
    TL_LAUNCH_CHECK("decay_scan");
    return TL_OK;
}

int tlb_head_norm_gate(const float *o, const void *w, float eps, const void *gate, long long g_token, int act, void *out, int tokens, int heads,
                       int dv, int dtype, void *stream) {
    if (tokens <= 0) return TL_OK;
    if (!o || !w || !out || heads <= 0 || dv <= 0 || act < 0 || act > 1) return tl::fail(TL_EINVAL, "head_norm_gate: bad argument");
    long long rows = (long long)tokens * heads;
    TLB_DISPATCH(dtype, "head_norm_gate",
                 head_norm_gate_kernel<T><<<(unsigned)((rows + 3) / 4), 128, 0, as_stream(stream)>>>(o, (const T *)w, eps, (const T *)gate, g_token, act,
                                                                                                    (T *)out, rows, heads, dv));
    TL_LAUNCH_CHECK("head_norm_gate");
    return TL_OK;
}

}  // extern "C"
