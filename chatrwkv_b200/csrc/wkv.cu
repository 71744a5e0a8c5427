// WKV state recurrences for RWKV-4 (scalar log-space state per channel) and RWKV-5 / RWKV-6
// (matrix state per head), sequence form.  All arithmetic is IEEE fp32 with accurate expf
// (the reference kernels are built with --use_fast_math; its pure-torch statement of the
// same recurrences, pkg/model.py:1069-1084 / 1245-1251 / 1327-1333, is the specification).
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------------
// RWKV-4: one thread per channel, sequential in t (reference: operators.cu:11-50).  k and v
// are fetched eight steps ahead of the dependent chain.
// ---------------------------------------------------------------------------------------
template <typename F>
__global__ void __launch_bounds__(32) wkv4_seq_kernel(int B, int T, int C,
                                                      const float* __restrict__ w_, const float* __restrict__ u_,
                                                      const F* __restrict__ k_, const F* __restrict__ v_,
                                                      F* __restrict__ y_, float* __restrict__ aa_,
                                                      float* __restrict__ bb_, float* __restrict__ pp_) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * C) return;
    const int b = idx / C, c = idx % C;
    const long long off = (long long)b * T * C + c;
    const F* k = k_ + off;
    const F* v = v_ + off;
    F* y = y_ + off;
    const float u = u_[c], w = w_[c];
    float aa = aa_[idx], bb = bb_[idx], pp = pp_[idx];
    constexpr int U = 8;
    int t = 0;
    for (; t + U <= T; t += U) {
        float kk[U], vv[U];
#pragma unroll
        for (int i = 0; i < U; ++i) {
            kk[i] = to_f32<F>(k[(long long)(t + i) * C]);
            vv[i] = to_f32<F>(v[(long long)(t + i) * C]);
        }
#pragma unroll
        for (int i = 0; i < U; ++i) {
            float ww = u + kk[i];
            float p = fmaxf(pp, ww);
            float e1 = expf(pp - p), e2 = expf(ww - p);
            y[(long long)(t + i) * C] = from_f32<F>((e1 * aa + e2 * vv[i]) / (e1 * bb + e2));
            ww = w + pp;
            p = fmaxf(ww, kk[i]);
            e1 = expf(ww - p); e2 = expf(kk[i] - p);
            aa = e1 * aa + e2 * vv[i];
            bb = e1 * bb + e2;
            pp = p;
        }
    }
    for (; t < T; ++t) {
        const float kk = to_f32<F>(k[(long long)t * C]), vv = to_f32<F>(v[(long long)t * C]);
        float ww = u + kk;
        float p = fmaxf(pp, ww);
        float e1 = expf(pp - p), e2 = expf(ww - p);
        y[(long long)t * C] = from_f32<F>((e1 * aa + e2 * vv) / (e1 * bb + e2));
        ww = w + pp;
        p = fmaxf(ww, kk);
        e1 = expf(ww - p); e2 = expf(kk - p);
        aa = e1 * aa + e2 * vv;
        bb = e1 * bb + e2;
        pp = p;
    }
    aa_[idx] = aa; bb_[idx] = bb; pp_[idx] = pp;
}

// ---------------------------------------------------------------------------------------
// RWKV-5 / RWKV-6 (reference: rwkv5.cu:8-72, rwkv6.cu:8-71).
// State S[h][i][j] (i = value index, j = key index).  A CTA owns one head and a slice of
// ROWS value indices; a thread owns (i, quarter of j): N/4 state values in registers, and
// the four quarters of y_t[i] = sum_j r[j] (u[j] k[j] v[i] + S[i][j]) meet by two shuffles.
// r, k, (w,) v of TC time steps are staged in shared memory per barrier pair.
// ---------------------------------------------------------------------------------------
constexpr int TC = 16;

template <typename F, int N, bool PER_TOKEN_W>
__global__ void __launch_bounds__(128) wkv56_seq_kernel(int T, int C, int H, float* __restrict__ state,
                                                        const F* __restrict__ r_, const F* __restrict__ k_,
                                                        const F* __restrict__ v_, const float* __restrict__ w_,
                                                        const F* __restrict__ u_, F* __restrict__ y_) {
    constexpr int JQ = 4, NJ = N / JQ;
    constexpr int ROWS = (N >= 32) ? 32 : N;       // value indices per CTA
    constexpr int THREADS = ROWS * JQ;
    const int slices = N / ROWS;
    const int h = blockIdx.x / slices, i0 = (blockIdx.x % slices) * ROWS;
    const int tid = threadIdx.x;
    if (tid >= THREADS) return;
    const int il = tid / JQ, jq = tid % JQ, i = i0 + il, jb = jq * NJ;

    __shared__ float sr[TC][N], sk[TC][N], sw[PER_TOKEN_W ? TC : 1][N], sv[TC][ROWS], su[N];

    float S[NJ];
    float* sp = state + ((long long)h * N + i) * N + jb;
#pragma unroll
    for (int j = 0; j < NJ; ++j) S[j] = sp[j];
    for (int j = tid; j < N; j += THREADS) {
        su[j] = to_f32<F>(u_[h * N + j]);
        if (!PER_TOKEN_W) sw[0][j] = w_[h * N + j];
    }

    for (int t0 = 0; t0 < T; t0 += TC) {
        const int nt = min(TC, T - t0);
        __syncthreads();
        for (int e = tid; e < nt * N; e += THREADS) {
            const int tt = e / N, j = e % N;
            const long long g = (long long)(t0 + tt) * C + h * N + j;
            sr[tt][j] = to_f32<F>(r_[g]);
            sk[tt][j] = to_f32<F>(k_[g]);
            if (PER_TOKEN_W) sw[tt][j] = w_[g];
        }
        for (int e = tid; e < nt * ROWS; e += THREADS) {
            const int tt = e / ROWS, ii = e % ROWS;
            sv[tt][ii] = to_f32<F>(v_[(long long)(t0 + tt) * C + h * N + i0 + ii]);
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float v = sv[tt][il];
            const float* wrow = PER_TOKEN_W ? sw[tt] : sw[0];
            float y = 0.f;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const float x = sk[tt][jb + j] * v;
                y = fmaf(sr[tt][jb + j], fmaf(su[jb + j], x, S[j]), y);
                S[j] = fmaf(S[j], wrow[jb + j], x);
            }
            y += __shfl_xor_sync(0xffffffffu, y, 1);
            y += __shfl_xor_sync(0xffffffffu, y, 2);
            if (jq == 0) y_[(long long)(t0 + tt) * C + h * N + i] = from_f32<F>(y);
        }
    }
#pragma unroll
    for (int j = 0; j < NJ; ++j) sp[j] = S[j];
}

template <typename F, bool PER_TOKEN_W>
int launch56(int T, int C, int H, float* state, const void* r, const void* k, const void* v,
             const float* w, const void* u, void* y, cudaStream_t st) {
    const int N = C / H;
#define RWKV_L56(NN)                                                                               \
    {                                                                                              \
        constexpr int ROWS = (NN >= 32) ? 32 : NN;                                                 \
        wkv56_seq_kernel<F, NN, PER_TOKEN_W><<<H * (NN / ROWS), ROWS * 4, 0, st>>>(               \
            T, C, H, state, (const F*)r, (const F*)k, (const F*)v, w, (const F*)u, (F*)y);        \
    }
    switch (N) {
    case 16: RWKV_L56(16) break;
    case 32: RWKV_L56(32) break;
    case 64: RWKV_L56(64) break;
    case 128: RWKV_L56(128) break;
    default: return RWKV_ERR_UNSUPPORTED;
    }
#undef RWKV_L56
    return rwkv_launch_status();
}

template <bool PER_TOKEN_W>
int forward56(int64_t B, int64_t T, int64_t C, int64_t H, float* state, const void* r, const void* k,
              const void* v, const float* w, const void* u, void* y, int dtype, void* stream) {
    RWKV_CHECK_ARG(B == 1 && T >= 1 && C >= 1 && H >= 1 && C % H == 0 && T * C <= (int64_t)INT32_MAX * 16);
    RWKV_CHECK_ARG(state && r && k && v && w && u && y);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
    case RWKV_F32: return launch56<float, PER_TOKEN_W>(int(T), int(C), int(H), state, r, k, v, w, u, y, st);
    case RWKV_F16: return launch56<__half, PER_TOKEN_W>(int(T), int(C), int(H), state, r, k, v, w, u, y, st);
    case RWKV_BF16: return launch56<__nv_bfloat16, PER_TOKEN_W>(int(T), int(C), int(H), state, r, k, v, w, u, y, st);
    default: return RWKV_ERR_INVALID_ARG;
    }
}

}  // namespace

extern "C" int rwkv_wkv4_forward(int64_t B, int64_t T, int64_t C, const float* w, const float* u,
                                 const void* k, const void* v, void* y, int kv_dtype,
                                 float* aa, float* bb, float* pp, void* stream) {
    RWKV_CHECK_ARG(B >= 1 && T >= 1 && C >= 1 && B * C <= INT32_MAX && T <= INT32_MAX);
    RWKV_CHECK_ARG(w && u && k && v && y && aa && bb && pp);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int blocks = int((B * C + 31) / 32);
    if (kv_dtype == RWKV_F16)
        wkv4_seq_kernel<__half><<<blocks, 32, 0, st>>>(int(B), int(T), int(C), w, u, (const __half*)k,
                                                       (const __half*)v, (__half*)y, aa, bb, pp);
    else if (kv_dtype == RWKV_F32)
        wkv4_seq_kernel<float><<<blocks, 32, 0, st>>>(int(B), int(T), int(C), w, u, (const float*)k,
                                                      (const float*)v, (float*)y, aa, bb, pp);
    else
        return RWKV_ERR_INVALID_ARG;
    return rwkv_launch_status();
}

extern "C" int rwkv_wkv5_forward(int64_t B, int64_t T, int64_t C, int64_t H, float* state,
                                 const void* r, const void* k, const void* v, const float* w, const void* u,
                                 void* y, int dtype, void* stream) {
    return forward56<false>(B, T, C, H, state, r, k, v, w, u, y, dtype, stream);
}

extern "C" int rwkv_wkv6_forward(int64_t B, int64_t T, int64_t C, int64_t H, float* state,
                                 const void* r, const void* k, const void* v, const float* w, const void* u,
                                 void* y, int dtype, void* stream) {
    return forward56<true>(B, T, C, H, state, r, k, v, w, u, y, dtype, stream);
}
