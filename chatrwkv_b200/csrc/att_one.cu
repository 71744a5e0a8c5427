// One-token pieces of the RWKV-5.2 / RWKV-6 attention block that are not matmuls over packed
// weights (att_one_v5_1 / att_one_v6_0, pkg/model.py:1157-1181, 1263-1298):
//   * the RWKV-6 data-dependent token shift: LayerNorm, xxx = xx + (sx - xx) * x_maa,
//     tanh(xxx @ tm_w1) (x) tm_w2 -> five mix offsets -> wx, kx, vx, rx, gx      (model.py:1264-1276)
//   * the RWKV-6 decay: w = exp(-exp(time_decay + tanh(wx @ td_w1) @ td_w2))     (model.py:1286-1287)
//   * the one-step WKV of v5/v6 on the [H, N, N] state, group-norm and the gate  (model.py:1289-1296)
// The two low-rank products share one pair of kernels: "lora_a" (a [D] vector times a [D, R]
// matrix, split over row slabs into fp32 partials) and "lora_b" (sum of the partials, tanh, the
// grouped [R/G] x [D] second factor and the pointwise tail).  Every fp16 torch op of the
// reference rounds once; r16() marks those places.
#include <cooperative_groups.h>

#include "common.cuh"
#include <algorithm>

namespace cg = cooperative_groups;

namespace {

constexpr int kT = 256;

__device__ __forceinline__ float block_sum(float v, float* sh8) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh8[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < int(blockDim.x >> 5); ++i) t += sh8[i];
    return t;
}

// Programmatic dependent launch: let the successor be scheduled, pull what does not depend on the
// predecessor toward L2, then wait for the predecessor.
__device__ __forceinline__ void pdl_open() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void l2_line(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

struct LoraA {
    int mode;               // 0: token shift from the residual stream; 1: the vector is given
    int D, R, slab;         // in-features, out-features, rows per CTA
    const __half* x;        // mode 0: residual stream [D]; mode 1: input vector [D]
    const __half* ln_w;     // mode 0
    const __half* ln_b;
    const __half* state;    // mode 0: previous token's LayerNorm output
    __half* new_state;      // mode 0: receives this token's LayerNorm output (may alias state)
    const __half* maa_x;    // mode 0
    const __half* w1;       // [D, R]
    float* partial;         // [R][slabs]
    __half* xx_out;         // mode 0: LayerNorm output [D]
    __half* d_out;          // mode 0: sx - xx [D]
};

// grid = slabs, block = 256.  Needs D % 8 == 0 and D <= 8192 in mode 0 (the vector lives in registers).
__global__ void __launch_bounds__(kT) lora_a_kernel(const LoraA a) {
    extern __shared__ float smem[];             // vin[slab] | part[nrs][R]
    __shared__ float sh8[kT / 32];
    float* vin = smem;
    float* part = smem + a.slab;
    const int tid = threadIdx.x;
    const int j0 = blockIdx.x * a.slab;
    const int nrows = min(a.slab, a.D - j0);
    pdl_open();
    {   // this CTA's rows of w1: nrows * R halfs, contiguous
        const char* base = reinterpret_cast<const char*>(a.w1 + (long long)j0 * a.R);
        const long long bytes = (long long)nrows * a.R * 2;
        for (long long o = (long long)tid * 128; o < bytes; o += (long long)kT * 128) l2_line(base + o);
    }
    pdl_wait();
    if (a.mode == 0) {
        uint4 xv4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j8 = (tid + i * kT) * 8;
            xv4[i] = j8 < a.D ? __ldcg(reinterpret_cast<const uint4*>(a.x) + (j8 >> 3)) : make_uint4(0, 0, 0, 0);
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2* h = reinterpret_cast<const __half2*>(&xv4[i]);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h[e]); s += f.x + f.y; }
        }
        const float mean = block_sum(s, sh8) / float(a.D);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if ((tid + i * kT) * 8 < a.D) {
                const __half2* h = reinterpret_cast<const __half2*>(&xv4[i]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h[e]);
                    q = fmaf(f.x - mean, f.x - mean, q);
                    q = fmaf(f.y - mean, f.y - mean, q);
                }
            }
        }
        const float rstd = rsqrtf(block_sum(q, sh8) / float(a.D) + 1e-5f);
        // rows of this slab, eight at a time (slabs start and end on multiples of 8): every operand
        // is fetched with one 16-byte load before anything is stored
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j8 = (tid + i * kT) * 8;
            if (j8 >= j0 && j8 < j0 + nrows) {
                const uint4 s4 = __ldcg(reinterpret_cast<const uint4*>(a.state) + (j8 >> 3));
                const uint4 w4 = __ldg(reinterpret_cast<const uint4*>(a.ln_w) + (j8 >> 3));
                const uint4 b4 = __ldg(reinterpret_cast<const uint4*>(a.ln_b) + (j8 >> 3));
                const uint4 m4 = __ldg(reinterpret_cast<const uint4*>(a.maa_x) + (j8 >> 3));
                const __half* hx = reinterpret_cast<const __half*>(&xv4[i]);
                const __half* hs = reinterpret_cast<const __half*>(&s4);
                const __half* hw = reinterpret_cast<const __half*>(&w4);
                const __half* hb = reinterpret_cast<const __half*>(&b4);
                const __half* hm = reinterpret_cast<const __half*>(&m4);
                uint4 xo, dq;
                __half* ho = reinterpret_cast<__half*>(&xo);
                __half* hd = reinterpret_cast<__half*>(&dq);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float xx = r16((__half2float(hx[e]) - mean) * rstd * __half2float(hw[e]) + __half2float(hb[e]));
                    const float dd = r16(__half2float(hs[e]) - xx);
                    vin[j8 + e - j0] = r16(xx + r16(dd * __half2float(hm[e])));
                    ho[e] = __float2half_rn(xx);
                    hd[e] = __float2half_rn(dd);
                }
                reinterpret_cast<uint4*>(a.xx_out)[j8 >> 3] = xo;
                reinterpret_cast<uint4*>(a.d_out)[j8 >> 3] = dq;
                reinterpret_cast<uint4*>(a.new_state)[j8 >> 3] = xo;
            }
        }
    } else {
        for (int l = tid; l < nrows; l += kT) vin[l] = __half2float(__ldcg(a.x + j0 + l));
    }
    __syncthreads();
    const int cpp = min(a.R, kT);               // columns per pass
    const int nrs = kT / cpp;                   // row splits
    const int c0 = tid % cpp, rs = tid / cpp;
    if (rs < nrs) {
        for (int c = c0; c < a.R; c += cpp) {
            float acc = 0.f;
            const __half* wp = a.w1 + (long long)(j0 + rs) * a.R + c;
            const long long stp = (long long)nrs * a.R;
            for (int l = rs; l < nrows; l += 16 * nrs, wp += 16 * stp) {       // 16 loads in flight, then the sums
                __half wv[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) wv[u] = (l + u * nrs < nrows) ? __ldg(wp + u * stp) : __half(0.f);
#pragma unroll
                for (int u = 0; u < 16; ++u) if (l + u * nrs < nrows) acc = fmaf(vin[l + u * nrs], __half2float(wv[u]), acc);
            }
            part[rs * a.R + c] = acc;
        }
    }
    __syncthreads();
    for (int c = tid; c < a.R; c += kT) {
        float s = 0.f;
        for (int q = 0; q < nrs; ++q) s += part[q * a.R + c];
        a.partial[(long long)c * gridDim.x + blockIdx.x] = s;     // [R][slabs]
    }
}

struct LoraB {
    int mode;               // 0: five token-shift mixes; 1: decay
    int D, R, G, slabs;     // G groups of R/G hidden units each
    const float* partial;   // [R][slabs]
    const __half* w2;       // [G][R/G][D]
    const __half* xx;       // mode 0 [D]
    const __half* dd;       // mode 0 [D]
    const __half* maa[5];   // mode 0: w, k, v, r, g
    __half* out[5];         // mode 0: wx, kx, vx, rx, gx
    const float* decay;     // mode 1 [D]
    float* w_out;           // mode 1 [D]: exp(-exp(decay + lora))
};

// grid = ceil(D / 64), block = 256; dynamic shared memory (R + 32 * G * 64) floats.  A CTA owns 64
// columns; thread (slice = tid / 8, chunk = tid % 8) multiplies the hidden units l = slice,
// slice + 32, ... of every group into eight adjacent columns (16-byte loads, all independent:
// one trip to memory), the 32 slices are added in order, and G * 64 threads-worth of outputs finish.
// Needs D % 8 == 0 and a 16-byte aligned w2.
__global__ void __launch_bounds__(kT) lora_b_kernel(const LoraB b) {
    extern __shared__ float h[];                // h[R] | accs[32][G][64]
    float* accs = h + b.R;
    const int tid = threadIdx.x;
    const int chunk = tid & 7, slice = tid >> 3;
    const int d0 = blockIdx.x * 64 + chunk * 8;
    const int L = b.R / b.G;
    pdl_open();
    for (int row = tid; row < b.R; row += kT)   // this CTA's 128-byte piece of every row of w2
        l2_line(b.w2 + (long long)row * b.D + blockIdx.x * 64);
    pdl_wait();
    for (int c = tid; c < b.R; c += kT) {
        const float* pp = b.partial + (long long)c * b.slabs;
        float s = 0.f;
        for (int p = 0; p < b.slabs; p += 16) {
            float pv[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) pv[u] = p + u < b.slabs ? __ldcg(pp + p + u) : 0.f;
#pragma unroll
            for (int u = 0; u < 16; ++u) s += pv[u];
        }
        h[c] = r16(tanhf(r16(s)));
    }
    __syncthreads();
    for (int f0 = 0; f0 < b.G; f0 += 5) {       // up to five groups at a time: their loads first
        float acc[5][8];
#pragma unroll
        for (int g = 0; g < 5; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
        for (int l = slice; l < L; l += 32) {
            uint4 wv[5];
#pragma unroll
            for (int g = 0; g < 5; ++g)
                wv[g] = (f0 + g < b.G && d0 < b.D) ? __ldg(reinterpret_cast<const uint4*>(b.w2 + ((long long)(f0 + g) * L + l) * b.D + d0))
                                                   : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int g = 0; g < 5; ++g) {
                if (f0 + g < b.G) {
                    const float hv = h[(f0 + g) * L + l];
                    const __half2* w2h = reinterpret_cast<const __half2*>(&wv[g]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 wf = __half22float2(w2h[e]);
                        acc[g][2 * e] = fmaf(hv, wf.x, acc[g][2 * e]);
                        acc[g][2 * e + 1] = fmaf(hv, wf.y, acc[g][2 * e + 1]);
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < 5; ++g)
            if (f0 + g < b.G)
#pragma unroll
                for (int e = 0; e < 8; ++e) accs[(slice * b.G + f0 + g) * 64 + chunk * 8 + e] = acc[g][e];
    }
    __syncthreads();
    for (int t = tid; t < b.G * 64; t += kT) {
        const int f = t >> 6, c = t & 63, d = blockIdx.x * 64 + c;
        if (d >= b.D) continue;
        float acc = 0.f;
#pragma unroll 8
        for (int sl = 0; sl < 32; ++sl) acc += accs[(sl * b.G + f) * 64 + c];
        const float m = r16(acc);
        if (b.mode == 0) {
            const float xx = __half2float(__ldcg(b.xx + d)), dd = __half2float(__ldcg(b.dd + d));
            b.out[f][d] = __float2half_rn(r16(xx + r16(dd * r16(__half2float(b.maa[f][d]) + m))));
        } else {
            b.w_out[d] = expf(-expf(b.decay[d] + m));
        }
    }
}

// One-step WKV of RWKV-5.2 / RWKV-6 for one token, then group-norm (eps 64e-5) and the gate.
// State in the model's layout [H, key j, value i] (pkg/model.py:1461-1471).  grid = H, block = 256:
// thread (q, i) covers the keys j = q, q + TPI, ... of value index i (TPI = 256 / N threads per i).
__global__ void __launch_bounds__(kT) wkv56_one_kernel(int N, const __half* __restrict__ r, const __half* __restrict__ k,
                                                      const __half* __restrict__ v, const float* __restrict__ w,
                                                      const float* __restrict__ u, const float* s_in, float* s_out,
                                                      const float* __restrict__ lnx_w, const float* __restrict__ lnx_b,
                                                      const __half* __restrict__ g, __half* __restrict__ out) {
    extern __shared__ float sm[];               // rr[N] kk[N] ww[N] uu[N] | acc[TPI][N]
    __shared__ float sh8[kT / 32];
    float* rr = sm; float* kk = sm + N; float* ww = sm + 2 * N; float* uu = sm + 3 * N; float* accs = sm + 4 * N;
    const int hh = blockIdx.x, tid = threadIdx.x, c0 = hh * N;
    pdl_open();
    {   // the head's state (written a token ago)
        const char* base = reinterpret_cast<const char*>(s_in + (long long)hh * N * N);
        for (long long o = (long long)tid * 128; o < (long long)N * N * 4; o += (long long)kT * 128) l2_line(base + o);
    }
    pdl_wait();
    for (int j = tid; j < N; j += kT) {
        rr[j] = __half2float(__ldcg(r + c0 + j));
        kk[j] = __half2float(__ldcg(k + c0 + j));
        ww[j] = __ldcg(w + c0 + j);
        uu[j] = u[c0 + j];
    }
    __syncthreads();
    const int TPI = max(1, kT / N);
    const int i = tid % N, q = tid / N;
    float acc = 0.f;
    if (q < TPI && tid < TPI * N) {
        const float vi = __half2float(__ldcg(v + c0 + i));
        const float* si = s_in + (long long)hh * N * N + i;
        float* so = s_out + (long long)hh * N * N + i;
        for (int jb = q; jb < N; jb += 16 * TPI) {      // 16 state values in flight, then the updates
            float sv[16];
#pragma unroll
            for (int t = 0; t < 16; ++t) sv[t] = jb + t * TPI < N ? __ldcg(si + (long long)(jb + t * TPI) * N) : 0.f;
#pragma unroll
            for (int t = 0; t < 16; ++t) {
                const int j = jb + t * TPI;
                if (j < N) {
                    const float a = kk[j] * vi;
                    acc = fmaf(rr[j], fmaf(uu[j], a, sv[t]), acc);
                    so[(long long)j * N] = fmaf(ww[j], sv[t], a);
                }
            }
        }
        accs[q * N + i] = acc;
    }
    __syncthreads();
    // y[i] for i = tid < N; then the statistics of the head's N values
    float y = 0.f;
    if (tid < N) for (int t = 0; t < TPI; ++t) y += accs[t * N + tid];
    const float mean = block_sum(tid < N ? y : 0.f, sh8) / float(N);
    const float dv = tid < N ? y - mean : 0.f;
    const float var = block_sum(dv * dv, sh8) / float(N);
    if (tid < N) {
        const int c = c0 + tid;
        const float o = dv * rsqrtf(var + 64e-5f) * lnx_w[c] + lnx_b[c];
        out[c] = __float2half_rn(r16(r16(o) * __half2float(__ldcg(g + c))));
    }
}

// ---------------------------------------------------------------------------------------------
// The token shift AND the decay of one RWKV-6 layer in ONE launch: a single cluster of 8 CTAs.
// Four dependent low-rank products need three all-to-all exchanges of a few hundred numbers;
// inside a cluster those are hardware barriers plus distributed-shared-memory loads (about a
// microsecond), while as separate launches every step paid a kernel boundary.  CTA r owns rows
// (and, for the second factors, columns) [r * rows, (r + 1) * rows) of the D channels, so the
// vector a stage needs is the one the same CTA produced in the stage before.  The other SMs
// stay free for the matmul launch that follows and is already filling its weight ring.
// ---------------------------------------------------------------------------------------------
constexpr int kPT = 512;

struct AttPre {
    int D, Lm, Ld, rows, ncta;   // ncta: CTAs of the one cluster (8, or 16 where the device allows it)
    int wsm;                     // 1: this CTA's slices of the four weight matrices are staged in shared memory
    const __half *x, *ln_w, *ln_b, *state, *maa_x, *w1, *w2, *dw1, *dw2;
    const __half* maa[5];
    const float* decay;
    __half *new_state, *xx_out, *d_out;
    __half* out[5];
    float* w_out;
};

__device__ __forceinline__ float block_sum512(float v, float* sh16) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh16[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kPT / 32; ++i) t += sh16[i];
    return t;
}

// part[c] = sum over this CTA's rows l of vin[l] * W[l][c]   (W row-major [nrows][R], R % 8 == 0)
template <bool SM>      // SM: W points into shared memory (plain loads) instead of global memory (read-only loads)
__device__ __forceinline__ void slab_gemv(const float* vin, int nrows, const __half* W, int R, float* red, float* part) {
    const int tid = threadIdx.x;
    const int cc = R >> 3, nrg = kPT / cc, rg = tid / cc, c = tid - rg * cc;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (rg < nrg) {
        for (int l0 = rg; l0 < nrows; l0 += 8 * nrg) {
            uint4 wv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int l = l0 + u * nrg;
                const uint4* src = reinterpret_cast<const uint4*>(W + (long long)l * R) + c;
                wv[u] = l < nrows ? (SM ? *src : __ldg(src)) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int l = l0 + u * nrg;
                if (l < nrows) {
                    const float hv = vin[l];
                    const __half2* w2h = reinterpret_cast<const __half2*>(&wv[u]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 wf = __half22float2(w2h[e]);
                        acc[2 * e] = fmaf(hv, wf.x, acc[2 * e]);
                        acc[2 * e + 1] = fmaf(hv, wf.y, acc[2 * e + 1]);
                    }
                }
            }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) red[rg * R + c * 8 + e] = acc[e];
    }
    __syncthreads();
    for (int c2 = tid; c2 < R; c2 += kPT) {
        float s = 0.f;
#pragma unroll 8
        for (int q = 0; q < nrg; ++q) s += red[q * R + c2];      // unrolled: the loads go out together, only the adds chain
        part[c2] = s;
    }
}

// For this CTA's columns d = j0 + l (l < ncols, ncols % 8 == 0) and every group f < G:
// fin(f, l, r16(sum over the group's hidden units u of h[f*L + u] * W2[f*L + u][d])).
template <bool SM, typename Fin>
__device__ __forceinline__ void cols_gemv(const float* h, int G, int L, const __half* W2, int D, int j0, int ncols, Fin fin) {
    const int tid = threadIdx.x, rs = tid & 7;
    const int nch = ncols >> 3;
    for (int cb = 0; cb < nch; cb += kPT / 8) {
        const int c = cb + (tid >> 3);
        const bool on = c < nch;
        for (int f = 0; f < G; ++f) {
            float acc[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = 0.f;
            if (on) {
                for (int l0 = rs; l0 < L; l0 += 64) {
                    uint4 wv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int l = l0 + 8 * u;
                        const uint4* src = reinterpret_cast<const uint4*>(W2 + ((long long)f * L + l) * D + j0) + c;
                        wv[u] = l < L ? (SM ? *src : __ldg(src)) : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int l = l0 + 8 * u;
                        if (l < L) {
                            const float hv = h[f * L + l];
                            const __half2* w2h = reinterpret_cast<const __half2*>(&wv[u]);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float2 wf = __half22float2(w2h[e]);
                                acc[2 * e] = fmaf(hv, wf.x, acc[2 * e]);
                                acc[2 * e + 1] = fmaf(hv, wf.y, acc[2 * e + 1]);
                            }
                        }
                    }
                }
            }
            float mine = 0.f;                   // the eight lanes of a chunk add up, lane rs keeps column rs
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float v = acc[e];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                if (e == rs) mine = v;
            }
            if (on) fin(f, c * 8 + rs, r16(mine));
        }
    }
}

__global__ void __launch_bounds__(kPT) v6_att_pre_kernel(const AttPre a) {
    extern __shared__ __align__(16) float sm[];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = int(cluster.block_rank());
    const int tid = threadIdx.x;
    const int R1 = 5 * a.Lm, R3 = a.Ld;
    const int Rm = max(R1, R3);
    float* vin = sm;                            // [rows]   xxx, later wx, of this CTA's channels
    float* xxs = vin + a.rows;                  // [rows]   LayerNorm output
    float* dds = xxs + a.rows;                  // [rows]   sx - xx
    float* part1 = dds + a.rows;                // [R1]     this CTA's share of xxx @ w1     (read by the cluster)
    float* part3 = part1 + R1;                  // [R3]     this CTA's share of wx @ dw1      (read by the cluster)
    float* h = part3 + R3;                      // [Rm]     tanh of the summed shares
    float* red = h + Rm;                        // [4096]   row-group sums
    __shared__ float sh16[kPT / 32];
    const int j0 = rank * a.rows;
    const int nrows = max(0, min(a.D, j0 + a.rows) - j0);     // multiple of 8
    // a.wsm: this CTA's slices of the weights in shared memory, fetched by cp.async while the LayerNorm runs:
    //   sw1 [nrows][R1] (later dw2's columns [R3][ld]), sw2 [R1][ld], sdw1 [nrows][R3];  ld = rows + 8 halves keeps
    //   the eight rows a warp reads at once on different banks.  Without it every stage paid one or more round
    //   trips to L2 / DRAM per group of rows (the launch cannot start early enough for a prefetch to land: a CTA of
    //   512 threads needs a whole SM's registers), 25 us per layer; with it the stages read shared memory.
    const int ld = a.rows + 8;
    __half* sw1 = reinterpret_cast<__half*>(red + 4096);
    __half* sw2 = sw1 + max(a.rows * R1, R3 * ld);
    __half* sdw1 = sw2 + R1 * ld;
    auto cp16 = [](void* dst, const void* src) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
    };
    // contiguous copy of `halves` fp16 values (a multiple of 8), and a copy of `nr` rows of `nrows` values each (the
    // row length in 16-byte pieces is a power of two for the usual D / 16 = 256: a shift instead of a division)
    auto copy_flat = [&](__half* dst, const __half* src, int halves) {
        for (int i = tid; i < (halves >> 3); i += kPT) cp16(dst + i * 8, src + i * 8);
    };
    auto copy_rows = [&](__half* dst, const __half* src, int nr, int src_ld, int dst_ld) {
        const int per = nrows >> 3;
        if ((per & (per - 1)) == 0 && per > 0) {
            const int sh = 31 - __clz(per);
            for (int i = tid; i < nr * per; i += kPT) {
                const int r = i >> sh, c = i & (per - 1);
                cp16(dst + (long long)r * dst_ld + c * 8, src + (long long)r * src_ld + c * 8);
            }
        } else {
            for (int i = tid; i < nr * per; i += kPT) {
                const int r = i / per, c = i - r * per;
                cp16(dst + (long long)r * dst_ld + c * 8, src + (long long)r * src_ld + c * 8);
            }
        }
    };
    auto commit = []() { asm volatile("cp.async.commit_group;" ::: "memory"); };
    // the per-channel constants of this CTA's rows and the previous token's vector, staged with the first group:
    // [ln w | ln b | maa x | state | maa 0..4] fp16 and [decay] fp32, `rows` entries each
    __half* svec = sdw1 + a.rows * R3;
    float* sdecay = reinterpret_cast<float*>(svec + 9 * a.rows);

    const bool dec = a.dw1 != nullptr;          // false: the token shift alone (the caller runs rwkv_v6_decay beside the matmuls)
    pdl_open();
    if (a.wsm) {
        copy_flat(sw1, a.w1 + (long long)j0 * R1, nrows * R1);
        copy_flat(svec, a.ln_w + j0, nrows);
        copy_flat(svec + a.rows, a.ln_b + j0, nrows);
        copy_flat(svec + 2 * a.rows, a.maa_x + j0, nrows);
        copy_flat(svec + 3 * a.rows, a.state + j0, nrows);
#pragma unroll
        for (int f = 0; f < 5; ++f) copy_flat(svec + (4 + f) * a.rows, a.maa[f] + j0, nrows);
        if (dec) copy_flat(reinterpret_cast<__half*>(sdecay), reinterpret_cast<const __half*>(a.decay + j0), nrows * 2);
        commit();
        copy_rows(sw2, a.w2 + j0, R1, a.D, ld);
        commit();
        if (dec) copy_flat(sdw1, a.dw1 + (long long)j0 * R3, nrows * R3);
        commit();                                                     // (an empty group keeps the wait counts below)
    } else {   // weights of this CTA, toward L2: its rows of w1 / dw1, its 16-byte column pieces of w2 / dw2
        const char* b1 = reinterpret_cast<const char*>(a.w1 + (long long)j0 * R1);
        for (long long o = (long long)tid * 128; o < (long long)nrows * R1 * 2; o += (long long)kPT * 128) l2_line(b1 + o);
        const char* b3 = reinterpret_cast<const char*>(a.dw1 + (long long)j0 * R3);
        for (long long o = (long long)tid * 128; dec && o < (long long)nrows * R3 * 2; o += (long long)kPT * 128) l2_line(b3 + o);
        const int lines = (nrows * 2 + 127) / 128;
        for (int i = tid; i < (R1 + (dec ? R3 : 0)) * lines; i += kPT) {
            const int row = i / lines, ln = i - row * lines;
            const __half* base = row < R1 ? a.w2 + (long long)row * a.D : a.dw2 + (long long)(row - R1) * a.D;
            l2_line(reinterpret_cast<const char*>(base + j0) + ln * 128);
        }
    }
    pdl_wait();

    // ---- LayerNorm of the whole vector; xx, dd, xxx for this CTA's channels (model.py:1264-1267)
    {
        uint4 xv4[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int j8 = (tid + i * kPT) * 8;
            xv4[i] = j8 < a.D ? __ldcg(reinterpret_cast<const uint4*>(a.x) + (j8 >> 3)) : make_uint4(0, 0, 0, 0);
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const __half2* hh = reinterpret_cast<const __half2*>(&xv4[i]);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(hh[e]); s += f.x + f.y; }
        }
        const float mean = block_sum512(s, sh16) / float(a.D);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if ((tid + i * kPT) * 8 < a.D) {
                const __half2* hh = reinterpret_cast<const __half2*>(&xv4[i]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(hh[e]);
                    q = fmaf(f.x - mean, f.x - mean, q);
                    q = fmaf(f.y - mean, f.y - mean, q);
                }
            }
        }
        if (a.wsm) asm volatile("cp.async.wait_group 2;" ::: "memory");     // the first group (w1, the vectors): the
        const float rstd = rsqrtf(block_sum512(q, sh16) / float(a.D) + 1e-5f);    // barriers of the sum publish them
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int j8 = (tid + i * kPT) * 8;
            if (j8 >= j0 && j8 < j0 + nrows) {
                uint4 s4, w4, b4, m4;
                if (a.wsm) {                     // staged before the wait (the first copy group has landed: see below)
                    const int o = j8 - j0;
                    w4 = *reinterpret_cast<const uint4*>(svec + o);
                    b4 = *reinterpret_cast<const uint4*>(svec + a.rows + o);
                    m4 = *reinterpret_cast<const uint4*>(svec + 2 * a.rows + o);
                    s4 = *reinterpret_cast<const uint4*>(svec + 3 * a.rows + o);
                } else {
                    s4 = __ldcg(reinterpret_cast<const uint4*>(a.state) + (j8 >> 3));
                    w4 = __ldg(reinterpret_cast<const uint4*>(a.ln_w) + (j8 >> 3));
                    b4 = __ldg(reinterpret_cast<const uint4*>(a.ln_b) + (j8 >> 3));
                    m4 = __ldg(reinterpret_cast<const uint4*>(a.maa_x) + (j8 >> 3));
                }
                const __half* hx = reinterpret_cast<const __half*>(&xv4[i]);
                const __half* hs = reinterpret_cast<const __half*>(&s4);
                const __half* hw = reinterpret_cast<const __half*>(&w4);
                const __half* hb = reinterpret_cast<const __half*>(&b4);
                const __half* hm = reinterpret_cast<const __half*>(&m4);
                uint4 xo, dq;
                __half* ho = reinterpret_cast<__half*>(&xo);
                __half* hd = reinterpret_cast<__half*>(&dq);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float xx = r16((__half2float(hx[e]) - mean) * rstd * __half2float(hw[e]) + __half2float(hb[e]));
                    const float dd = r16(__half2float(hs[e]) - xx);
                    const int l = j8 + e - j0;
                    vin[l] = r16(xx + r16(dd * __half2float(hm[e])));
                    xxs[l] = xx;
                    dds[l] = dd;
                    ho[e] = __float2half_rn(xx);
                    hd[e] = __float2half_rn(dd);
                }
                reinterpret_cast<uint4*>(a.xx_out)[j8 >> 3] = xo;
                reinterpret_cast<uint4*>(a.d_out)[j8 >> 3] = dq;
                reinterpret_cast<uint4*>(a.new_state)[j8 >> 3] = xo;
            }
        }
    }
    __syncthreads();

    // ---- xxx @ w1 -> tanh -> five offsets -> wx, kx, vx, rx, gx (model.py:1268-1276) ----------
    if (a.wsm) {
        asm volatile("cp.async.wait_group 2;" ::: "memory");         // w1 has landed
        __syncthreads();
        slab_gemv<true>(vin, nrows, sw1, R1, red, part1);
        if (dec) copy_rows(sw1, a.dw2 + j0, R3, a.D, ld);            // w1's room is free: dw2's columns go there
        commit();
    } else {
        slab_gemv<false>(vin, nrows, a.w1 + (long long)j0 * R1, R1, red, part1);
    }
    cluster.sync();
    for (int c = tid; c < R1; c += kPT) {
        float s = 0.f;
        for (int q = 0; q < a.ncta; ++q) s += cluster.map_shared_rank(part1, q)[c];
        h[c] = r16(tanhf(r16(s)));
    }
    auto mix_out = [&](int f, int l, float m) {
        const float mf = __half2float(a.wsm ? svec[(4 + f) * a.rows + l] : a.maa[f][j0 + l]);
        const float v = r16(xxs[l] + r16(dds[l] * r16(mf + m)));
        a.out[f][j0 + l] = __float2half_rn(v);
        if (f == 0) vin[l] = v;                 // wx: the input of the decay product
    };
    if (a.wsm) {
        asm volatile("cp.async.wait_group 2;" ::: "memory");         // w2 has landed (dw1, dw2 may still be on their way)
        __syncthreads();
        cols_gemv<true>(h, 5, a.Lm, sw2, ld, 0, nrows, mix_out);
    } else {
        __syncthreads();
        cols_gemv<false>(h, 5, a.Lm, a.w2, a.D, j0, nrows, mix_out);
    }
    if (!dec) {
        cluster.sync();                         // nobody leaves while its share of the first product is being read
        return;
    }
    __syncthreads();

    // ---- w = exp(-exp(time_decay + tanh(wx @ dw1) @ dw2)) (model.py:1286-1287) ---------------
    if (a.wsm) {
        asm volatile("cp.async.wait_group 1;" ::: "memory");         // dw1 has landed
        __syncthreads();
        slab_gemv<true>(vin, nrows, sdw1, R3, red, part3);
    } else {
        slab_gemv<false>(vin, nrows, a.dw1 + (long long)j0 * R3, R3, red, part3);
    }
    cluster.sync();
    for (int c = tid; c < R3; c += kPT) {
        float s = 0.f;
        for (int q = 0; q < a.ncta; ++q) s += cluster.map_shared_rank(part3, q)[c];
        h[c] = r16(tanhf(r16(s)));
    }
    auto decay_out = [&](int, int l, float m) { a.w_out[j0 + l] = expf(-expf((a.wsm ? sdecay[l] : a.decay[j0 + l]) + m)); };
    if (a.wsm) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");         // dw2 has landed
        __syncthreads();
        cols_gemv<true>(h, 1, a.Ld, sw1, ld, 0, nrows, decay_out);
    } else {
        __syncthreads();
        cols_gemv<false>(h, 1, a.Ld, a.dw2, a.D, j0, nrows, decay_out);
    }
    cluster.sync();                             // nobody leaves while its shares are being read
}

}  // namespace

static inline int lora_slab(int64_t D) { return D >= 4096 ? 128 : (D >= 1024 ? 64 : 32); }

extern "C" size_t rwkv_v6_scratch_bytes(int64_t D, int64_t rank) {
    if (D < 1 || rank < 1) return 0;
    const int slab = lora_slab(D);
    return size_t((D + slab - 1) / slab) * size_t(rank) * sizeof(float);
}

extern "C" int rwkv_v6_token_shift(int64_t D, int64_t Lm, const void* x, const void* state, void* new_state,
                                   const void* ln_w, const void* ln_b,
                                   const void* maa_x, const void* const* maa5, const void* tm_w1, const void* tm_w2,
                                   float* scratch, size_t scratch_bytes, void* xx_out, void* d_out, void* const* out5,
                                   void* stream) {
    RWKV_CHECK_ARG(D >= 8 && D % 8 == 0 && D <= 8 * 4 * kT && Lm >= 1 && 5 * Lm <= 1024);
    RWKV_CHECK_ARG(x && state && new_state && ln_w && ln_b && maa_x && maa5 && tm_w1 && tm_w2 && scratch && xx_out && d_out && out5);
    RWKV_CHECK_ALIGN(x, 16); RWKV_CHECK_ALIGN(state, 16); RWKV_CHECK_ALIGN(new_state, 16); RWKV_CHECK_ALIGN(ln_w, 16);
    RWKV_CHECK_ALIGN(ln_b, 16); RWKV_CHECK_ALIGN(maa_x, 16); RWKV_CHECK_ALIGN(tm_w2, 16); RWKV_CHECK_ALIGN(xx_out, 16); RWKV_CHECK_ALIGN(d_out, 16);
    const int R = int(5 * Lm);
    const int slab = lora_slab(D);
    const int slabs = int((D + slab - 1) / slab);
    if (scratch_bytes < size_t(slabs) * R * sizeof(float)) return RWKV_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LoraA a = {};
    a.mode = 0; a.D = int(D); a.R = R; a.slab = slab;
    a.x = static_cast<const __half*>(x); a.ln_w = static_cast<const __half*>(ln_w); a.ln_b = static_cast<const __half*>(ln_b);
    a.state = static_cast<const __half*>(state); a.new_state = static_cast<__half*>(new_state); a.maa_x = static_cast<const __half*>(maa_x);
    a.w1 = static_cast<const __half*>(tm_w1); a.partial = scratch;
    a.xx_out = static_cast<__half*>(xx_out); a.d_out = static_cast<__half*>(d_out);
    const int nrs = kT / (R < kT ? R : kT);
    if (int rc = rwkv_launch_pdl(lora_a_kernel, dim3(slabs), dim3(kT), (slab + nrs * R) * sizeof(float), st, a)) return rc;
    LoraB b = {};
    b.mode = 0; b.D = int(D); b.R = R; b.G = 5; b.slabs = slabs; b.partial = scratch;
    b.w2 = static_cast<const __half*>(tm_w2); b.xx = a.xx_out; b.dd = a.d_out;
    for (int f = 0; f < 5; ++f) {
        RWKV_CHECK_ARG(maa5[f] && out5[f]);
        b.maa[f] = static_cast<const __half*>(maa5[f]);
        b.out[f] = static_cast<__half*>(out5[f]);
    }
    return rwkv_launch_pdl(lora_b_kernel, dim3(int((D + 63) / 64)), dim3(kT), (R + 32 * b.G * 64) * sizeof(float), st, b);
}

extern "C" int rwkv_v6_decay(int64_t D, int64_t Ld, const void* wx, const void* td_w1, const void* td_w2,
                             const float* time_decay, float* scratch, size_t scratch_bytes, float* w_out, void* stream) {
    RWKV_CHECK_ARG(D >= 8 && D % 8 == 0 && Ld >= 1 && Ld <= 4096);
    RWKV_CHECK_ALIGN(td_w2, 16);
    RWKV_CHECK_ARG(wx && td_w1 && td_w2 && time_decay && scratch && w_out);
    const int R = int(Ld);
    const int slab = lora_slab(D);
    const int slabs = int((D + slab - 1) / slab);
    if (scratch_bytes < size_t(slabs) * R * sizeof(float)) return RWKV_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LoraA a = {};
    a.mode = 1; a.D = int(D); a.R = R; a.slab = slab;
    a.x = static_cast<const __half*>(wx); a.w1 = static_cast<const __half*>(td_w1); a.partial = scratch;
    const int nrs = kT / (R < kT ? R : kT);
    if (int rc = rwkv_launch_pdl(lora_a_kernel, dim3(slabs), dim3(kT), (slab + nrs * R) * sizeof(float), st, a)) return rc;
    LoraB b = {};
    b.mode = 1; b.D = int(D); b.R = R; b.G = 1; b.slabs = slabs; b.partial = scratch;
    b.w2 = static_cast<const __half*>(td_w2); b.decay = time_decay; b.w_out = w_out;
    return rwkv_launch_pdl(lora_b_kernel, dim3(int((D + 63) / 64)), dim3(kT), (R + 32 * b.G * 64) * sizeof(float), st, b);
}

extern "C" int rwkv_wkv56_one(int64_t H, int64_t N, const void* r, const void* k, const void* v, const float* w,
                              const float* u, const float* state, float* new_state, const float* lnx_w,
                              const float* lnx_b, const void* g, void* out, void* stream) {
    RWKV_CHECK_ARG(H >= 1 && H <= 65535 && N >= 1 && N <= kT);
    RWKV_CHECK_ARG(r && k && v && w && u && state && new_state && lnx_w && lnx_b && g && out);
    const int TPI = kT / int(N) > 0 ? kT / int(N) : 1;
    return rwkv_launch_pdl(wkv56_one_kernel, dim3(int(H)), dim3(kT), (4 * N + TPI * N) * sizeof(float),
                           static_cast<cudaStream_t>(stream), int(N), static_cast<const __half*>(r),
                           static_cast<const __half*>(k), static_cast<const __half*>(v), w, u, state, new_state, lnx_w, lnx_b,
                           static_cast<const __half*>(g), static_cast<__half*>(out));
}

// Token shift + decay of one RWKV-6 layer in one single-cluster launch (see v6_att_pre_kernel).
// RWKV_ERR_UNSUPPORTED when the shapes do not fit it (ranks not multiples of 8, D > 8192): the
// caller then uses rwkv_v6_token_shift followed by rwkv_v6_decay, which compute the same values.
extern "C" int rwkv_v6_att_pre(int64_t D, int64_t Lm, int64_t Ld, const void* x, const void* state, void* new_state,
                               const void* ln_w, const void* ln_b, const void* maa_x, const void* const* maa5,
                               const void* tm_w1, const void* tm_w2, const void* td_w1, const void* td_w2,
                               const float* time_decay, void* xx_out, void* d_out, void* const* out5, float* w_out,
                               void* stream) {
    RWKV_CHECK_ARG(D >= 8 && D % 8 == 0 && Lm >= 1 && Ld >= 1);
    RWKV_CHECK_ARG(x && state && new_state && ln_w && ln_b && maa_x && maa5 && tm_w1 && tm_w2 && xx_out && d_out && out5);
    // the four decay arguments all given, or all NULL: the token shift alone, rwkv_v6_decay to follow
    const bool with_decay = td_w1 != nullptr;
    RWKV_CHECK_ARG((td_w2 != nullptr) == with_decay && (time_decay != nullptr) == with_decay && (w_out != nullptr) == with_decay);
    if (D > 8 * 2 * kPT || (5 * Lm) % 8 != 0 || Ld % 8 != 0 || 5 * Lm > 1024 || Ld > 1024) return RWKV_ERR_UNSUPPORTED;
    const void* al[] = {x, state, new_state, ln_w, ln_b, maa_x, tm_w1, tm_w2, td_w1, td_w2, xx_out, d_out};
    for (const void* p : al) RWKV_CHECK_ALIGN(p, 16);            // (NULL passes)
    AttPre a = {};
    a.D = int(D); a.Lm = int(Lm); a.Ld = int(Ld);
    // 16 CTAs (a non-portable cluster size) halve every CTA's share of the weights; 8 where the
    // device or the shape (fewer than 16 x 8 channels) does not allow it.
    static int big_by_device[64];            // 0 = not asked yet, 1 = allowed, 2 = refused (function attributes are per device)
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); dev = -1; }
    int big = dev >= 0 ? big_by_device[dev] : 0;
    if (big == 0) {
        big = cudaFuncSetAttribute(v6_att_pre_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess ? 1 : 2;
        if (dev >= 0) big_by_device[dev] = big;
    }
    cudaGetLastError();
    a.ncta = (big == 1 && D >= 16 * 64) ? 16 : 8;
    a.rows = int(((D + a.ncta - 1) / a.ncta + 7) / 8 * 8);
    a.x = static_cast<const __half*>(x); a.ln_w = static_cast<const __half*>(ln_w); a.ln_b = static_cast<const __half*>(ln_b);
    a.state = static_cast<const __half*>(state); a.maa_x = static_cast<const __half*>(maa_x);
    a.w1 = static_cast<const __half*>(tm_w1); a.w2 = static_cast<const __half*>(tm_w2);
    a.dw1 = static_cast<const __half*>(td_w1); a.dw2 = static_cast<const __half*>(td_w2);
    a.decay = time_decay;
    a.new_state = static_cast<__half*>(new_state); a.xx_out = static_cast<__half*>(xx_out); a.d_out = static_cast<__half*>(d_out);
    a.w_out = w_out;
    for (int f = 0; f < 5; ++f) {
        RWKV_CHECK_ARG(maa5[f] && out5[f]);
        a.maa[f] = static_cast<const __half*>(maa5[f]);
        a.out[f] = static_cast<__half*>(out5[f]);
    }
    const int R1 = int(5 * Lm), R3 = int(Ld);
    const size_t work = size_t(3 * a.rows + R1 + R3 + (R1 > R3 ? R1 : R3) + 4096) * sizeof(float);
    if (work > 48 * 1024) return RWKV_ERR_UNSUPPORTED;
    // the CTA's weight slices in shared memory when they fit next to the working arrays (RWKV_B200_V6_PRE_SMEM=0: never)
    auto weights_bytes = [&](int rows) {
        const size_t ldw = size_t(rows) + 8;
        return (std::max(size_t(rows) * R1, size_t(R3) * ldw) + size_t(R1) * ldw + size_t(rows) * R3 + 9 * size_t(rows)) * sizeof(__half) +
               size_t(rows) * sizeof(float);
    };
    static int use_wsm = -1;
    if (use_wsm < 0) { const char* e = getenv("RWKV_B200_V6_PRE_SMEM"); use_wsm = (e != nullptr && e[0] == '0') ? 0 : 1; }
    static bool big_smem[64] = {};           // the opt-in to more than 48 KB is per device
    a.wsm = (use_wsm && work + weights_bytes(a.rows) <= 226 * 1024) ? 1 : 0;
    if (a.wsm && dev >= 0 && !big_smem[dev]) {
        if (cudaFuncSetAttribute(v6_att_pre_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) {
            cudaGetLastError();
            a.wsm = 0;
        } else {
            big_smem[dev] = true;
        }
    }
    if (dev < 0) a.wsm = 0;
    size_t smem = work + (a.wsm ? weights_bytes(a.rows) : 0);
    static int use_pdl = -1;
    if (use_pdl < 0) {
        const char* e = getenv("RWKV_B200_PDL");
        use_pdl = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(a.ncta));
    cfg.blockDim = dim3(kPT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = unsigned(a.ncta);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, v6_att_pre_kernel, a);
    if (e != cudaSuccess && a.ncta == 16) {      // no room for a 16-CTA cluster: 8 from now on
        cudaGetLastError();
        big = 0;
        a.ncta = 8;
        a.rows = int(((D + 7) / 8 + 7) / 8 * 8);
        a.wsm = (a.wsm && work + weights_bytes(a.rows) <= 226 * 1024) ? 1 : 0;
        smem = work + (a.wsm ? weights_bytes(a.rows) : 0);
        cfg.dynamicSmemBytes = smem;
        cfg.gridDim = dim3(8);
        attr[0].val.clusterDim.x = 8;
        e = cudaLaunchKernelEx(&cfg, v6_att_pre_kernel, a);
    }
    if (e != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    return RWKV_OK;
}
