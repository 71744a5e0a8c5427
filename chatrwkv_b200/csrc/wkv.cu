// WKV state recurrences for RWKV-4 (scalar log-space state per channel) and RWKV-5 / RWKV-6
// (matrix state per head), sequence form.  All arithmetic is IEEE fp32 with accurate expf
// (the reference kernels are built with --use_fast_math; its pure-torch statement of the
// same recurrences, pkg/model.py:1069-1084 / 1245-1251 / 1327-1333, is the specification).
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------------
// RWKV-4 (the recurrence of operators.cu:30-46 / pkg/model.py:1069-1084), parallel in time.
//
// Per channel the state is (aa, bb, pp): A = aa e^pp = sum_s e^{(t-1-s) w + k_s} v_s and B likewise
// without v.  A step multiplies A, B by e^w and adds e^{k_t} (v_t, 1): an affine map, so T steps
// split into chunks of Lc: (1) every (chunk, channel) runs its Lc steps from the empty state and
// keeps the chunk's own sums (a_c, b_c, p_c); (2) every (chunk, channel) folds the summaries of the
// chunks before it into the caller's state -- state' = e^{w Lc} state + summary, in the same
// max-shifted form as a step -- and then (3) runs its Lc steps again from that state, now writing
// y.  Twice the arithmetic, T / Lc times the threads: 1024 tokens x 4096 channels keep 131072
// threads busy instead of 4096, each with 32 dependent steps instead of 1024.  With one chunk
// (T <= Lc) only the second kernel runs and nothing is recomputed.
// MULR: y is multiplied by r (the receptance) with the reference's roundings, y -> dtype, then
// r * y -> dtype (cuda_att_seq, pkg/model.py:1359-1360).
// ---------------------------------------------------------------------------------------
constexpr int kWkv4Threads = 128;
constexpr int kWkv4MaxChunks = 64;

struct Wkv4State { float aa, bb, pp; };

__device__ __forceinline__ void wkv4_step(Wkv4State& s, float w, float kk, float vv) {
    const float ww = w + s.pp;
    const float p = fmaxf(ww, kk);
    const float e1 = expf(ww - p), e2 = expf(kk - p);
    s.aa = e1 * s.aa + e2 * vv;
    s.bb = e1 * s.bb + e2;
    s.pp = p;
}

// summaries of chunks 0 .. NC-2 (the last chunk's is never needed) and a copy of the caller's state
template <typename F>
__global__ void __launch_bounds__(kWkv4Threads) wkv4_summary_kernel(int T, int C, int Lc, int NC, const float* __restrict__ w_,
                                                                    const F* __restrict__ k_, const F* __restrict__ v_,
                                                                    const float* __restrict__ aa_, const float* __restrict__ bb_,
                                                                    const float* __restrict__ pp_, float* __restrict__ summ,
                                                                    float* __restrict__ init) {
    const int c = blockIdx.x * kWkv4Threads + threadIdx.x, chunk = blockIdx.y, b = blockIdx.z;
    if (c >= C) return;
    if (chunk == 0) {
        float* ini = init + (size_t)b * 3 * C;
        ini[c] = aa_[(size_t)b * C + c]; ini[C + c] = bb_[(size_t)b * C + c]; ini[2 * C + c] = pp_[(size_t)b * C + c];
    }
    const float w = w_[c];
    const int t0 = chunk * Lc, t1 = min(T, t0 + Lc);
    const F* k = k_ + ((size_t)b * T + t0) * C + c;
    const F* v = v_ + ((size_t)b * T + t0) * C + c;
    Wkv4State s = {0.f, 0.f, -1e30f};
    const int n = t1 - t0;
    int t = 0;
    for (; t + 4 <= n; t += 4) {
        float kk[4], vv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { kk[i] = to_f32<F>(k[(size_t)(t + i) * C]); vv[i] = to_f32<F>(v[(size_t)(t + i) * C]); }
#pragma unroll
        for (int i = 0; i < 4; ++i) wkv4_step(s, w, kk[i], vv[i]);
    }
    for (; t < n; ++t) wkv4_step(s, w, to_f32<F>(k[(size_t)t * C]), to_f32<F>(v[(size_t)t * C]));
    float* out = summ + ((size_t)b * NC + chunk) * 3 * C;
    out[c] = s.aa; out[C + c] = s.bb; out[2 * C + c] = s.pp;
}

template <typename F, bool MULR>
__global__ void __launch_bounds__(kWkv4Threads) wkv4_apply_kernel(int T, int C, int Lc, int NC, const float* __restrict__ w_,
                                                                  const float* __restrict__ u_, const F* __restrict__ k_,
                                                                  const F* __restrict__ v_, const F* __restrict__ r_, F* __restrict__ y_,
                                                                  float* aa_, float* bb_, float* pp_,
                                                                  const float* __restrict__ summ, const float* __restrict__ init) {
    const int c = blockIdx.x * kWkv4Threads + threadIdx.x, chunk = blockIdx.y, b = blockIdx.z;
    if (c >= C) return;
    const float w = w_[c], u = u_[c];
    Wkv4State s;
    if (NC == 1) {
        s.aa = aa_[(size_t)b * C + c]; s.bb = bb_[(size_t)b * C + c]; s.pp = pp_[(size_t)b * C + c];
    } else {
        const float* ini = init + (size_t)b * 3 * C;
        s.aa = ini[c]; s.bb = ini[C + c]; s.pp = ini[2 * C + c];
        const float wl = w * float(Lc);
        for (int j = 0; j < chunk; ++j) {       // state after chunk j = e^{w Lc} state + summary_j
            const float* sm = summ + ((size_t)b * NC + j) * 3 * C;
            const float sa = sm[c], sb = sm[C + c], sp = sm[2 * C + c];
            const float ww = wl + s.pp;
            const float p = fmaxf(ww, sp);
            const float e1 = expf(ww - p), e2 = expf(sp - p);
            s.aa = e1 * s.aa + e2 * sa;
            s.bb = e1 * s.bb + e2 * sb;
            s.pp = p;
        }
    }
    const int t0 = chunk * Lc, t1 = min(T, t0 + Lc);
    const size_t base = ((size_t)b * T + t0) * C + c;
    const F* k = k_ + base;
    const F* v = v_ + base;
    const F* r = MULR ? r_ + base : nullptr;
    F* y = y_ + base;
    const int n = t1 - t0;
    int t = 0;
    for (; t + 4 <= n; t += 4) {
        float kk[4], vv[4], rr[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            kk[i] = to_f32<F>(k[(size_t)(t + i) * C]); vv[i] = to_f32<F>(v[(size_t)(t + i) * C]);
            rr[i] = MULR ? to_f32<F>(r[(size_t)(t + i) * C]) : 1.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float ww = u + kk[i];
            const float p = fmaxf(s.pp, ww);
            const float e1 = expf(s.pp - p), e2 = expf(ww - p);
            const float yv = (e1 * s.aa + e2 * vv[i]) / (e1 * s.bb + e2);
            y[(size_t)(t + i) * C] = MULR ? from_f32<F>(rr[i] * to_f32<F>(from_f32<F>(yv))) : from_f32<F>(yv);
            wkv4_step(s, w, kk[i], vv[i]);
        }
    }
    for (; t < n; ++t) {
        const float kk = to_f32<F>(k[(size_t)t * C]), vv = to_f32<F>(v[(size_t)t * C]);
        const float ww = u + kk;
        const float p = fmaxf(s.pp, ww);
        const float e1 = expf(s.pp - p), e2 = expf(ww - p);
        const float yv = (e1 * s.aa + e2 * vv) / (e1 * s.bb + e2);
        y[(size_t)t * C] = MULR ? from_f32<F>(to_f32<F>(r[(size_t)t * C]) * to_f32<F>(from_f32<F>(yv))) : from_f32<F>(yv);
        wkv4_step(s, w, kk, vv);
    }
    if (chunk == NC - 1) { aa_[(size_t)b * C + c] = s.aa; bb_[(size_t)b * C + c] = s.bb; pp_[(size_t)b * C + c] = s.pp; }
}

static inline void wkv4_chunks(int64_t T, int& Lc, int& NC) {
    Lc = T <= 32 * kWkv4MaxChunks ? 32 : int((T + kWkv4MaxChunks - 1) / kWkv4MaxChunks);
    NC = int((T + Lc - 1) / Lc);
}

// ---------------------------------------------------------------------------------------
// RWKV-5 / RWKV-6 (the recurrences of rwkv5.cu:32-68, rwkv6.cu:30-67 / pkg/model.py:1245-1251, 1324-1333).
// State S[h][i][j] (i = value index, j = key index):
//     y_t[i] = sum_j r_t[j] (u[j] k_t[j] v_t[i] + S[i][j]);   S[i][j] <- w_t[j] S[i][j] + k_t[j] v_t[i]
// A CTA owns one head; its N x N state lives in the registers of (N / TL)^2 threads as TL x TL tiles (see
// Wkv56Tile).  r, k, v (, w) of TC time steps are staged in shared memory per barrier pair.
//
// Parallel in time (more than one chunk): S_t is affine in S_{t-1}, so (1) every chunk runs its steps
// from S = 0 and keeps its own sum and the product P[j] of its decays (PASS_SUM); (2) a scan kernel
// turns the sums into the state at the start of every chunk, S <- P (.) S + sum, chunk after chunk
// (64 cheap steps instead of T); (3) every chunk runs its steps again from that state and writes y
// (PASS_OUT).  No division by decay products, so decays that underflow to 0 are harmless.
// `model_layout`: the caller's state is [h][j][i] (the transpose: what RWKV.forward keeps in its state
// list, pkg/model.py:1376, 1384) instead of the operator's [h][i][j].
// ---------------------------------------------------------------------------------------
constexpr int TC = 16;
constexpr int kWkv56MaxChunks = 16;
enum { PASS_WHOLE = 0, PASS_SUM = 1, PASS_OUT = 2 };

struct Wkv56Args {
    int T, C, H, Lc, NC, model_layout;
    int vec;                // r, k, v, w allow 16-byte copies
    const float* state;     // the caller's state
    float* state_out;       // where the new state goes (PASS_WHOLE, last chunk of PASS_OUT); may be `state`
    float* sums;            // [NC][H][N][N]: PASS_SUM writes chunk sums; the scan leaves the state after chunk c in [c]
    float* prods;           // [NC][H][N]
    float* start;           // [H][N][N] copy of the caller's state in operator layout (made by the scan)
};

// Thread tile of the N x N state: TL x TL values in registers (8 x 8 for the usual N = 64: 64 threads per
// head).  Per step a thread reads r, k, w of its TL key indices and v of its TL value indices from shared
// memory (4 * TL words for 3 * TL * TL multiply-adds), and
//     y[i] = sum_j r[j] S[i][j] + v[i] * sum_j r[j] u[j] k[j]
// is completed across the N / TL threads that share a value index by log2(N / TL) shuffles.
template <int N> struct Wkv56Tile { static constexpr int TL = N >= 64 ? 8 : N >= 32 ? 4 : 2; static constexpr int NT = N / TL; };

template <int N, int TL>
__device__ __forceinline__ long long wkv56_state_index(int model_layout, int h, int i, int j) {
    return model_layout ? ((long long)h * N + j) * N + i : ((long long)h * N + i) * N + j;
}

__device__ __forceinline__ void cp16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
template <typename F> __device__ __forceinline__ float2 load_pair(const F* p);
template <> __device__ __forceinline__ float2 load_pair<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <> __device__ __forceinline__ float2 load_pair<__half>(const __half* p) { return __half22float2(*reinterpret_cast<const __half2*>(p)); }
template <> __device__ __forceinline__ float2 load_pair<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// Two fp32 multiply-adds / multiplies per instruction (sm_100); each lane rounds as fmaf / a product does.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)),
          "l"(reinterpret_cast<const unsigned long long&>(c)));
    return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)));
    return d;
}

template <typename FI, typename FO, int N, bool PER_TOKEN_W, int PASS>
__global__ void __launch_bounds__(Wkv56Tile<N>::NT * Wkv56Tile<N>::NT)
wkv56_seq_kernel(const Wkv56Args a, const FI* __restrict__ r_, const FI* __restrict__ k_, const FI* __restrict__ v_,
                 const float* __restrict__ w_, const FO* __restrict__ u_, FO* __restrict__ y_) {
    constexpr int TL = Wkv56Tile<N>::TL, NT = Wkv56Tile<N>::NT, THREADS = NT * NT;
    const int C = a.C, h = blockIdx.x, chunk = blockIdx.y, tid = threadIdx.x;
    const int ti = tid / NT, tj = tid % NT, i0 = ti * TL, j0 = tj * TL;
    const int t_begin = PASS == PASS_WHOLE ? 0 : chunk * a.Lc;
    const int t_end = PASS == PASS_WHOLE ? a.T : min(a.T, t_begin + a.Lc);

    // r, k, v (and the per-token decay) of TCN steps at a time, in the caller's dtype, double-buffered: the next
    // block's 16-byte cp.async copies are in flight while this block's steps run
    constexpr int TCN = N >= 128 ? TC / 2 : TC;
    __shared__ __align__(16) FI sr[2][TCN][N], sk[2][TCN][N], sv[2][TCN][N];
    __shared__ __align__(16) float sw[2][PER_TOKEN_W ? TCN : 1][N];

    float2 S2[TL][TL / 2], P2[TL / 2], u2[TL / 2];       // the state tile, the decay product and u as pairs along j
    const float* src = PASS == PASS_OUT ? (chunk == 0 ? a.start : a.sums + (long long)(chunk - 1) * a.H * N * N) : a.state;
    const int src_layout = PASS == PASS_OUT ? 0 : a.model_layout;
    auto stage = [&](int t0, int buf) {
        const int nt = min(TCN, t_end - t0);
        if (a.vec) {
            constexpr int CI = N * int(sizeof(FI)) / 16, CW = N * 4 / 16;         // 16-byte pieces per row
            for (int e = tid; e < nt * CI; e += THREADS) {
                const int tt = e / CI, c = e - tt * CI;
                const long long g = ((long long)(t0 + tt) * C + h * N) * (long long)sizeof(FI) + c * 16;
                cp16(reinterpret_cast<uint8_t*>(&sr[buf][tt][0]) + c * 16, reinterpret_cast<const uint8_t*>(r_) + g);
                cp16(reinterpret_cast<uint8_t*>(&sk[buf][tt][0]) + c * 16, reinterpret_cast<const uint8_t*>(k_) + g);
                cp16(reinterpret_cast<uint8_t*>(&sv[buf][tt][0]) + c * 16, reinterpret_cast<const uint8_t*>(v_) + g);
            }
            if (PER_TOKEN_W)
                for (int e = tid; e < nt * CW; e += THREADS) {
                    const int tt = e / CW, c = e - tt * CW;
                    cp16(reinterpret_cast<uint8_t*>(&sw[buf][tt][0]) + c * 16,
                         reinterpret_cast<const uint8_t*>(w_) + ((long long)(t0 + tt) * C + h * N) * 4 + c * 16);
                }
        } else {
            for (int e = tid; e < nt * N; e += THREADS) {
                const int tt = e / N, j = e % N;
                const long long g = (long long)(t0 + tt) * C + h * N + j;
                sr[buf][tt][j] = r_[g];
                sk[buf][tt][j] = k_[g];
                sv[buf][tt][j] = v_[g];
                if (PER_TOKEN_W) sw[buf][tt][j] = w_[g];
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (t_begin < t_end) stage(t_begin, 0);
#pragma unroll
    for (int q = 0; q < TL / 2; ++q) {
        P2[q] = make_float2(1.f, 1.f);
        u2[q] = make_float2(to_f32<FO>(u_[h * N + j0 + 2 * q]), to_f32<FO>(u_[h * N + j0 + 2 * q + 1]));
    }
#pragma unroll
    for (int ii = 0; ii < TL; ++ii)
#pragma unroll
        for (int q = 0; q < TL / 2; ++q) {
            S2[ii][q].x = PASS == PASS_SUM ? 0.f : src[wkv56_state_index<N, TL>(src_layout, h, i0 + ii, j0 + 2 * q)];
            S2[ii][q].y = PASS == PASS_SUM ? 0.f : src[wkv56_state_index<N, TL>(src_layout, h, i0 + ii, j0 + 2 * q + 1)];
        }
    if (!PER_TOKEN_W)
        for (int j = tid; j < N; j += THREADS) sw[0][0][j] = sw[1][0][j] = w_[h * N + j];

    int buf = 0;
    for (int t0 = t_begin; t0 < t_end; t0 += TCN, buf ^= 1) {
        const int nt = min(TCN, t_end - t0);
        if (t0 + TCN < t_end) {
            stage(t0 + TCN, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            // operands as pairs: the multiply-adds below are two-wide fp32 instructions (same roundings as fmaf)
            float2 r2[TL / 2], k2[TL / 2], w2[TL / 2];
            float v[TL];
            const float* wrow = PER_TOKEN_W ? sw[buf][tt] : sw[0][0];
#pragma unroll
            for (int q = 0; q < TL / 2; ++q) {
                r2[q] = load_pair<FI>(&sr[buf][tt][j0 + 2 * q]);
                k2[q] = load_pair<FI>(&sk[buf][tt][j0 + 2 * q]);
                w2[q] = *reinterpret_cast<const float2*>(&wrow[j0 + 2 * q]);
            }
#pragma unroll
            for (int q = 0; q < TL / 2; ++q) {
                const float2 vp = load_pair<FI>(&sv[buf][tt][i0 + 2 * q]);
                v[2 * q] = vp.x;
                v[2 * q + 1] = vp.y;
            }
            if (PASS != PASS_SUM) {
                float2 ruk2 = make_float2(0.f, 0.f);
#pragma unroll
                for (int q = 0; q < TL / 2; ++q) ruk2 = ffma2(fmul2(r2[q], u2[q]), k2[q], ruk2);
                const float ruk = ruk2.x + ruk2.y;
                float y[TL];
#pragma unroll
                for (int ii = 0; ii < TL; ++ii) {
                    float2 acc = make_float2(v[ii] * ruk, 0.f);
#pragma unroll
                    for (int q = 0; q < TL / 2; ++q) acc = ffma2(r2[q], S2[ii][q], acc);
                    y[ii] = acc.x + acc.y;
                }
                // sum over the NT threads of a row of tiles: whole exchanges while there are more lanes than values,
                // then halving exchanges (each lane keeps half of what it holds), so that lane tj ends with y[tj]
#pragma unroll
                for (int o = NT >> 1; o >= TL; o >>= 1) {
#pragma unroll
                    for (int ii = 0; ii < TL; ++ii) y[ii] += __shfl_xor_sync(0xffffffffu, y[ii], o);
                }
#pragma unroll
                for (int o = (TL < NT ? TL : NT) >> 1; o > 0; o >>= 1) {
                    const bool upper = (tj & o) != 0;
#pragma unroll
                    for (int q = 0; q < o; ++q) {
                        const float send = upper ? y[q] : y[q + o];
                        const float keep = upper ? y[q + o] : y[q];
                        y[q] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                    }
                }
                if (tj < TL) y_[(long long)(t0 + tt) * C + h * N + i0 + tj] = from_f32<FO>(y[0]);
            }
#pragma unroll
            for (int ii = 0; ii < TL; ++ii) {
                const float2 vv = make_float2(v[ii], v[ii]);
#pragma unroll
                for (int q = 0; q < TL / 2; ++q) S2[ii][q] = ffma2(S2[ii][q], w2[q], fmul2(k2[q], vv));
            }
            if (PASS == PASS_SUM) {
#pragma unroll
                for (int q = 0; q < TL / 2; ++q) P2[q] = fmul2(P2[q], w2[q]);
            }
        }
        __syncthreads();                                 // this block's buffer is refilled two rounds on
    }
    if (PASS == PASS_SUM) {
        float* out = a.sums + (long long)chunk * a.H * N * N;
#pragma unroll
        for (int ii = 0; ii < TL; ++ii)
#pragma unroll
            for (int q = 0; q < TL / 2; ++q) {
                out[wkv56_state_index<N, TL>(0, h, i0 + ii, j0 + 2 * q)] = S2[ii][q].x;
                out[wkv56_state_index<N, TL>(0, h, i0 + ii, j0 + 2 * q + 1)] = S2[ii][q].y;
            }
        if (ti == 0) {
#pragma unroll
            for (int q = 0; q < TL / 2; ++q) {
                a.prods[((long long)chunk * a.H + h) * N + j0 + 2 * q] = P2[q].x;
                a.prods[((long long)chunk * a.H + h) * N + j0 + 2 * q + 1] = P2[q].y;
            }
        }
    } else if (PASS == PASS_WHOLE || chunk == a.NC - 1) {
#pragma unroll
        for (int ii = 0; ii < TL; ++ii)
#pragma unroll
            for (int q = 0; q < TL / 2; ++q) {
                a.state_out[wkv56_state_index<N, TL>(a.model_layout, h, i0 + ii, j0 + 2 * q)] = S2[ii][q].x;
                a.state_out[wkv56_state_index<N, TL>(a.model_layout, h, i0 + ii, j0 + 2 * q + 1)] = S2[ii][q].y;
            }
    }
}

// start <- the caller's state (operator layout); sums[c] <- state after chunk c, for c = 0 .. NC - 2.
// One thread per state element; every load of the chain is issued before the first multiply-add.
template <int N>
__global__ void __launch_bounds__(256) wkv56_scan_kernel(const Wkv56Args a) {
    const int h = blockIdx.x;
    const int e = blockIdx.y * 256 + threadIdx.x;
    if (e >= N * N) return;
    const int i = e / N, j = e % N;
    const long long at = ((long long)h * N + i) * N + j;
    float add[kWkv56MaxChunks], mul[kWkv56MaxChunks];
#pragma unroll
    for (int c = 0; c < kWkv56MaxChunks - 1; ++c) {
        const bool on = c + 1 < a.NC;
        add[c] = on ? a.sums[(long long)c * a.H * N * N + at] : 0.f;
        mul[c] = on ? a.prods[((long long)c * a.H + h) * N + j] : 1.f;
    }
    float S = a.state[wkv56_state_index<N, 1>(a.model_layout, h, i, j)];
    a.start[at] = S;
#pragma unroll
    for (int c = 0; c < kWkv56MaxChunks - 1; ++c) {
        if (c + 1 < a.NC) {
            S = fmaf(S, mul[c], add[c]);
            a.sums[(long long)c * a.H * N * N + at] = S;
        }
    }
}

static inline void wkv56_chunks(int64_t T, int& Lc, int& NC) {
    // chunks of 128 steps, at most 16 of them: every pass then has a few CTAs per SM, and the steps a CTA runs
    // one after the other stay a small multiple of what the parallel passes cost
    Lc = T <= 128 * kWkv56MaxChunks ? 128 : int((T + kWkv56MaxChunks - 1) / kWkv56MaxChunks);
    Lc = (Lc + TC - 1) / TC * TC;
    NC = int((T + Lc - 1) / Lc);
}

static inline size_t wkv56_ws_bytes(int64_t T, int64_t C, int64_t H) {
    int Lc, NC;
    wkv56_chunks(T, Lc, NC);
    if (NC == 1) return 0;
    const size_t N = size_t(C / H);
    return (size_t(NC) * size_t(H) * N * N + size_t(NC) * size_t(H) * N + size_t(H) * N * N) * sizeof(float);
}

template <typename FI, typename FO, bool PER_TOKEN_W>
int launch56(int T, int C, int H, const float* state, float* state_out, const void* r, const void* k, const void* v,
             const float* w, const void* u, void* y, int model_layout, void* workspace, size_t workspace_bytes, cudaStream_t st) {
    const int N = C / H;
    Wkv56Args a;
    a.T = T; a.C = C; a.H = H; a.model_layout = model_layout; a.state = state; a.state_out = state_out;
    a.vec = ((reinterpret_cast<uintptr_t>(r) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
              reinterpret_cast<uintptr_t>(w)) % 16 == 0 && (size_t(C) * sizeof(FI)) % 16 == 0 && (size_t(N) * sizeof(FI)) % 16 == 0) ? 1 : 0;
    wkv56_chunks(T, a.Lc, a.NC);
    if (a.NC > 1 && (workspace == nullptr || workspace_bytes < wkv56_ws_bytes(T, C, H))) { a.NC = 1; a.Lc = T; }
    a.sums = static_cast<float*>(workspace);
    a.prods = a.NC > 1 ? a.sums + (size_t)a.NC * H * N * N : nullptr;
    a.start = a.NC > 1 ? a.prods + (size_t)a.NC * H * N : nullptr;
#define RWKV_L56(NN)                                                                                          \
    {                                                                                                         \
        constexpr int THR = Wkv56Tile<NN>::NT * Wkv56Tile<NN>::NT;                                            \
        const unsigned gx = unsigned(H);                                                                      \
        if (a.NC == 1) {                                                                                      \
            wkv56_seq_kernel<FI, FO, NN, PER_TOKEN_W, PASS_WHOLE><<<gx, THR, 0, st>>>(                       \
                a, (const FI*)r, (const FI*)k, (const FI*)v, w, (const FO*)u, (FO*)y);                        \
        } else {                                                                                              \
            wkv56_seq_kernel<FI, FO, NN, PER_TOKEN_W, PASS_SUM><<<dim3(gx, unsigned(a.NC - 1)), THR, 0, st>>>( \
                a, (const FI*)r, (const FI*)k, (const FI*)v, w, (const FO*)u, (FO*)y);                        \
            wkv56_scan_kernel<NN><<<dim3(gx, unsigned((NN * NN + 255) / 256)), 256, 0, st>>>(a);                                                     \
            wkv56_seq_kernel<FI, FO, NN, PER_TOKEN_W, PASS_OUT><<<dim3(gx, unsigned(a.NC)), THR, 0, st>>>(    \
                a, (const FI*)r, (const FI*)k, (const FI*)v, w, (const FO*)u, (FO*)y);                        \
        }                                                                                                     \
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

// in_dtype: r, k, v; out_dtype: u, y (the reference's operators use one dtype for all five)
template <bool PER_TOKEN_W>
int forward56(int64_t B, int64_t T, int64_t C, int64_t H, const float* state, float* state_out, const void* r, const void* k,
              const void* v, const float* w, const void* u, void* y, int in_dtype, int out_dtype, int model_layout,
              void* workspace, size_t workspace_bytes, void* stream) {
    RWKV_CHECK_ARG(B == 1 && T >= 1 && C >= 1 && H >= 1 && C % H == 0 && T * C <= (int64_t)INT32_MAX * 16);
    RWKV_CHECK_ARG(state && state_out && r && k && v && w && u && y);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define RWKV_F56(FI, FO) return launch56<FI, FO, PER_TOKEN_W>(int(T), int(C), int(H), state, state_out, r, k, v, w, u, y, model_layout, workspace, workspace_bytes, st)
    if (in_dtype == RWKV_F32 && out_dtype == RWKV_F32) RWKV_F56(float, float);
    if (in_dtype == RWKV_F16 && out_dtype == RWKV_F16) RWKV_F56(__half, __half);
    if (in_dtype == RWKV_BF16 && out_dtype == RWKV_BF16) RWKV_F56(__nv_bfloat16, __nv_bfloat16);
    if (in_dtype == RWKV_F16 && out_dtype == RWKV_F32) RWKV_F56(__half, float);
#undef RWKV_F56
    return RWKV_ERR_INVALID_ARG;
}

}  // namespace

extern "C" size_t rwkv_wkv4_workspace_bytes(int64_t B, int64_t T, int64_t C) {
    if (B < 1 || T < 1 || C < 1) return 0;
    int Lc, NC;
    wkv4_chunks(T, Lc, NC);
    return NC == 1 ? 0 : size_t(B) * size_t(NC + 1) * 3 * size_t(C) * sizeof(float);
}

template <typename F>
static int wkv4_launch(int64_t B, int64_t T, int64_t C, const float* w, const float* u, const F* k, const F* v, const F* r, F* y,
                       float* aa, float* bb, float* pp, void* workspace, size_t workspace_bytes, cudaStream_t st) {
    int Lc, NC;
    wkv4_chunks(T, Lc, NC);
    if (NC > 1 && (workspace == nullptr || workspace_bytes < rwkv_wkv4_workspace_bytes(B, T, C))) { Lc = int(T); NC = 1; }   // one chunk: sequential
    float* summ = static_cast<float*>(workspace);
    float* init = NC > 1 ? summ + size_t(B) * NC * 3 * C : nullptr;
    const dim3 grid((unsigned)((C + kWkv4Threads - 1) / kWkv4Threads), (unsigned)NC, (unsigned)B);
    if (NC > 1) {
        const dim3 g1(grid.x, (unsigned)(NC - 1), grid.z);
        wkv4_summary_kernel<F><<<g1, kWkv4Threads, 0, st>>>(int(T), int(C), Lc, NC, w, k, v, aa, bb, pp, summ, init);
    }
    if (r != nullptr)
        wkv4_apply_kernel<F, true><<<grid, kWkv4Threads, 0, st>>>(int(T), int(C), Lc, NC, w, u, k, v, r, y, aa, bb, pp, summ, init);
    else
        wkv4_apply_kernel<F, false><<<grid, kWkv4Threads, 0, st>>>(int(T), int(C), Lc, NC, w, u, k, v, r, y, aa, bb, pp, summ, init);
    return rwkv_launch_status();
}

extern "C" int rwkv_wkv4_seq(int64_t B, int64_t T, int64_t C, const float* w, const float* u,
                             const void* k, const void* v, const void* r, void* y, int kv_dtype,
                             float* aa, float* bb, float* pp, void* workspace, size_t workspace_bytes, void* stream) {
    RWKV_CHECK_ARG(B >= 1 && T >= 1 && C >= 1 && B <= 65535 && B * C <= INT32_MAX && T <= INT32_MAX);
    RWKV_CHECK_ARG(w && u && k && v && y && aa && bb && pp);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (kv_dtype == RWKV_F16)
        return wkv4_launch<__half>(B, T, C, w, u, (const __half*)k, (const __half*)v, (const __half*)r, (__half*)y, aa, bb, pp,
                                   workspace, workspace_bytes, st);
    if (kv_dtype == RWKV_F32)
        return wkv4_launch<float>(B, T, C, w, u, (const float*)k, (const float*)v, (const float*)r, (float*)y, aa, bb, pp,
                                  workspace, workspace_bytes, st);
    return RWKV_ERR_INVALID_ARG;
}

extern "C" int rwkv_wkv4_forward(int64_t B, int64_t T, int64_t C, const float* w, const float* u,
                                 const void* k, const void* v, void* y, int kv_dtype,
                                 float* aa, float* bb, float* pp, void* stream) {
    return rwkv_wkv4_seq(B, T, C, w, u, k, v, nullptr, y, kv_dtype, aa, bb, pp, nullptr, 0, stream);
}

extern "C" int rwkv_wkv5_forward(int64_t B, int64_t T, int64_t C, int64_t H, float* state,
                                 const void* r, const void* k, const void* v, const float* w, const void* u,
                                 void* y, int dtype, void* stream) {
    return forward56<false>(B, T, C, H, state, state, r, k, v, w, u, y, dtype, dtype, 0, nullptr, 0, stream);
}

extern "C" int rwkv_wkv6_forward(int64_t B, int64_t T, int64_t C, int64_t H, float* state,
                                 const void* r, const void* k, const void* v, const float* w, const void* u,
                                 void* y, int dtype, void* stream) {
    return forward56<true>(B, T, C, H, state, state, r, k, v, w, u, y, dtype, dtype, 0, nullptr, 0, stream);
}

extern "C" size_t rwkv_wkv56_workspace_bytes(int64_t T, int64_t C, int64_t H) {
    if (T < 1 || C < 1 || H < 1 || C % H != 0) return 0;
    return wkv56_ws_bytes(T, C, H);
}

extern "C" int rwkv_wkv56_seq(int per_token_w, int64_t T, int64_t C, int64_t H, const float* state, float* state_out, int model_layout,
                              const void* r, const void* k, const void* v, const float* w, const void* u, void* y,
                              int in_dtype, int out_dtype, void* workspace, size_t workspace_bytes, void* stream) {
    return per_token_w ? forward56<true>(1, T, C, H, state, state_out, r, k, v, w, u, y, in_dtype, out_dtype, model_layout, workspace, workspace_bytes, stream)
                       : forward56<false>(1, T, C, H, state, state_out, r, k, v, w, u, y, in_dtype, out_dtype, model_layout, workspace, workspace_bytes, stream);
}
