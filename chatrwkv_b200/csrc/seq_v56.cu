// Pointwise pieces of the RWKV-5.2 / RWKV-6 sequence steps (cuda_att_seq_v5_2 / cuda_att_seq_v6_0 with
// v6_0_before and v5_2_after, pkg/model.py:1379-1439), one launch each; every torch op on fp16 tensors in
// the reference rounds once to fp16, r16() marks the same rounding points.
#include "common.cuh"

namespace {

constexpr int kPw = 256;

// The five data-dependent token-shift mixes of RWKV-6 for T rows:
//   sx_t = (t == 0 ? state : xx_{t-1}) - xx_t;  out_j[t] = xx_t + sx_t * (maa_j + m_j[t])     j = w, k, v, r, g
// (pkg/model.py:1407, 1414-1420); m = the low-rank product [5, T, D].  state_stride != 0: every row is a
// sequence of its own with its previous token's xx at state + t * state_stride (batched decode).
__global__ void __launch_bounds__(kPw) v6_seq_mix_kernel(int T, int D, const __half* __restrict__ xx, long long xx_stride,
                                                         const __half* __restrict__ state, long long state_stride,
                                                         const __half* __restrict__ m,
                                                         const __half* m0, const __half* m1, const __half* m2, const __half* m3,
                                                         const __half* m4, __half* o0, __half* o1, __half* o2, __half* o3, __half* o4) {
    const long long idx = (long long)blockIdx.x * kPw + threadIdx.x;       // over T * D / 2 pairs
    const int D2 = D >> 1;
    if (idx >= (long long)T * D2) return;
    const int t = int(idx / D2), d = int(idx % D2) * 2;
    const __half2 cur = *reinterpret_cast<const __half2*>(xx + (long long)t * xx_stride + d);
    const __half2 prev = (t == 0 || state_stride != 0) ? *reinterpret_cast<const __half2*>(state + t * state_stride + d)
                                : *reinterpret_cast<const __half2*>(xx + (long long)(t - 1) * xx_stride + d);
    const __half2 sx = __hsub2(prev, cur);
    const __half* maa[5] = {m0, m1, m2, m3, m4};
    __half* out[5] = {o0, o1, o2, o3, o4};
#pragma unroll
    for (int j = 0; j < 5; ++j) {
        const __half2 mj = *reinterpret_cast<const __half2*>(m + ((long long)j * T + t) * D + d);
        const __half2 a = __hadd2(*reinterpret_cast<const __half2*>(maa[j] + d), mj);
        *reinterpret_cast<__half2*>(out[j] + (long long)t * D + d) = __hadd2(cur, __hmul2(sx, a));
    }
}

// out[g][t][r] = tanh(in[t][g][r]): the [T, 5, Lm] -> [5, T, Lm] regrouping of pkg/model.py:1412 in the same pass
__global__ void __launch_bounds__(kPw) tanh_f16_kernel(long long n, int T, int G, int R, const __half* __restrict__ in,
                                                       __half* __restrict__ out) {
    const long long i = (long long)blockIdx.x * kPw + threadIdx.x;
    if (i >= n) return;
    const int r = int(i % R), g = int((i / R) % G);
    const long long t = i / ((long long)R * G);
    out[((long long)g * T + t) * R + r] = __float2half_rn(tanhf(__half2float(in[i])));
}

// per-token decay of RWKV-6: exp(-exp(time_decay + float(d2)))  (pkg/model.py:1422 and :959)
__global__ void __launch_bounds__(kPw) v6_seq_decay_kernel(long long n, int D, const float* __restrict__ decay,
                                                           const __half* __restrict__ d2, float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * kPw + threadIdx.x;
    if (i < n) out[i] = expf(-expf(decay[i % D] + __half2float(d2[i])));
}

// group-norm over each head's N channels (biased variance, eps), ln_x weight and bias in fp32, one rounding to
// fp16, then the gate product in fp16 (pkg/model.py:1386-1388).  One warp per (row, head).
__global__ void __launch_bounds__(kPw) v56_seq_gn_gate_kernel(int T, int H, int N, const float* __restrict__ y,
                                                              const float* __restrict__ lw, const float* __restrict__ lb,
                                                              const __half* __restrict__ g, __half* __restrict__ out, float eps) {
    const long long wid = ((long long)blockIdx.x * kPw + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)T * H) return;
    const int h = int(wid % H);
    const long long base = wid * N;            // (t * H + h) * N
    float v[4];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int n = lane + 32 * i;
        v[i] = n < N ? y[base + n] : 0.f;
        s += v[i];
    }
    const float mean = warp_sum(s) / float(N);
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int n = lane + 32 * i;
        const float c = n < N ? v[i] - mean : 0.f;
        q = fmaf(c, c, q);
    }
    const float rstd = rsqrtf(warp_sum(q) / float(N) + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int n = lane + 32 * i;
        if (n < N) {
            const float o = r16((v[i] - mean) * rstd * lw[h * N + n] + lb[h * N + n]);
            out[base + n] = __float2half_rn(o * __half2float(g[base + n]));
        }
    }
}

}  // namespace

extern "C" int rwkv_v6_seq_mix(int64_t T, int64_t D, const void* xx, int64_t xx_stride, const void* state, int64_t state_stride,
                               const void* m, const void* const* maa5, void* const* out5, void* stream) {
    RWKV_CHECK_ARG(T >= 1 && D >= 2 && D % 2 == 0 && xx && state && m && maa5 && out5 && xx_stride >= D && xx_stride % 2 == 0 &&
                   state_stride % 2 == 0);
    for (int j = 0; j < 5; ++j) RWKV_CHECK_ARG(maa5[j] != nullptr && out5[j] != nullptr);
    const long long n = T * (D / 2);
    v6_seq_mix_kernel<<<(unsigned)((n + kPw - 1) / kPw), kPw, 0, static_cast<cudaStream_t>(stream)>>>(
        int(T), int(D), (const __half*)xx, xx_stride, (const __half*)state, state_stride, (const __half*)m, (const __half*)maa5[0],
        (const __half*)maa5[1], (const __half*)maa5[2], (const __half*)maa5[3], (const __half*)maa5[4], (__half*)out5[0],
        (__half*)out5[1], (__half*)out5[2], (__half*)out5[3], (__half*)out5[4]);
    return rwkv_launch_status();
}

extern "C" int rwkv_tanh_regroup_f16(int64_t T, int64_t G, int64_t R, const void* in, void* out, void* stream) {
    RWKV_CHECK_ARG(T >= 1 && G >= 1 && R >= 1 && in && out && (G == 1 || in != out));
    const long long n = T * G * R;
    tanh_f16_kernel<<<(unsigned)((n + kPw - 1) / kPw), kPw, 0, static_cast<cudaStream_t>(stream)>>>(n, int(T), int(G), int(R),
                                                                                                  (const __half*)in, (__half*)out);
    return rwkv_launch_status();
}

extern "C" int rwkv_v6_seq_decay(int64_t T, int64_t D, const float* time_decay, const void* d2, float* out, void* stream) {
    RWKV_CHECK_ARG(T >= 1 && D >= 1 && time_decay && d2 && out);
    const long long n = T * D;
    v6_seq_decay_kernel<<<(unsigned)((n + kPw - 1) / kPw), kPw, 0, static_cast<cudaStream_t>(stream)>>>(n, int(D), time_decay,
                                                                                                      (const __half*)d2, out);
    return rwkv_launch_status();
}

extern "C" int rwkv_v56_seq_gn_gate(int64_t T, int64_t H, int64_t N, const float* y, const float* ln_w, const float* ln_b,
                                    const void* g, void* out, float eps, void* stream) {
    RWKV_CHECK_ARG(T >= 1 && H >= 1 && N >= 1 && N <= 128 && y && ln_w && ln_b && g && out);
    const long long threads = T * H * 32;
    v56_seq_gn_gate_kernel<<<(unsigned)((threads + kPw - 1) / kPw), kPw, 0, static_cast<cudaStream_t>(stream)>>>(
        int(T), int(H), int(N), y, ln_w, ln_b, (const __half*)g, (__half*)out, eps);
    return rwkv_launch_status();
}
