// Pointwise pieces of the att / ffn steps, fused into single launches: LayerNorm + token
// shift mixes (reference: the first lines of att_one / att_seq / ffn_one / ffn_seq and their
// v6 forms, pkg/model.py:984-1029, 1034-1038, 1263-1276) and the RWKV-4 one-step WKV update
// (pkg/model.py:1044-1055).  Every torch op on fp16 tensors in the reference rounds once to
// fp16; r16() marks the same rounding points here.
#include "common.cuh"
#include <algorithm>

namespace {

constexpr int kLnThreads = 256;
constexpr int kLnMaxPer = 32;   // D <= 8192

__device__ __forceinline__ float block_sum(float v, float* sh) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kLnThreads / 32; ++i) t += sh[i];
    return t;
}

// LayerNorm of one row held in registers: fp32 statistics, one rounding of the result.
template <int PER>
__device__ __forceinline__ void layer_norm_row(const __half* __restrict__ x, int D, const __half* __restrict__ w,
                                               const __half* __restrict__ b, float (&out)[PER], float* sh) {
    float v[PER];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = threadIdx.x + i * kLnThreads;
        v[i] = d < D ? __half2float(x[d]) : 0.f;
        s += v[i];
    }
    const float mean = block_sum(s, sh) / float(D);
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = threadIdx.x + i * kLnThreads;
        const float c = d < D ? v[i] - mean : 0.f;
        q = fmaf(c, c, q);
    }
    const float rstd = rsqrtf(block_sum(q, sh) / float(D) + 1e-5f);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = threadIdx.x + i * kLnThreads;
        out[i] = d < D ? r16((v[i] - mean) * rstd * __half2float(w[d]) + __half2float(b[d])) : 0.f;
    }
}

struct LnMixArgs {
    const __half* x; long long x_stride;      // [T, D]
    const __half* sx;                          // [D] previous token's LayerNorm output (state)
    long long sx_stride;                       // 0: the rows are consecutive tokens of one sequence; else row t is a
                                               // sequence of its own whose previous token's output is sx + t * sx_stride
    const __half* ln_w; const __half* ln_b;
    const __half* mix[5];                      // [D] each (or [T, D] when mix_stride != 0)
    long long mix_stride;
    __half* out[5]; long long out_stride;      // [T, D] each
    __half* xx_out; long long xx_stride;       // optional [T, D]: the LayerNorm output itself
    __half* new_state;                         // [D]: LayerNorm output of the last row
    int T, D, n_mix, mode;
};

// mode 0 (RWKV-4/5):  out = xx*mix + sx*(1-mix)      (pkg/model.py:986, 1036)
// mode 1 (RWKV-6):    out = xx + (sx-xx)*mix         (pkg/model.py:1009-1011, 1272)
template <int PER>
__global__ void __launch_bounds__(kLnThreads) ln_mix_kernel(const LnMixArgs a) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float sh[kLnThreads / 32];
    const int t = blockIdx.x;
    float xx[PER], prev[PER];
    layer_norm_row<PER>(a.x + (long long)t * a.x_stride, a.D, a.ln_w, a.ln_b, xx, sh);
    if (a.n_mix > 0) {
        if (t == 0 || a.sx_stride != 0) {
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int d = threadIdx.x + i * kLnThreads;
                prev[i] = d < a.D ? __half2float(a.sx[(long long)t * a.sx_stride + d]) : 0.f;
            }
        } else {
            layer_norm_row<PER>(a.x + (long long)(t - 1) * a.x_stride, a.D, a.ln_w, a.ln_b, prev, sh);
        }
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = threadIdx.x + i * kLnThreads;
        if (d >= a.D) continue;
        if (a.xx_out) a.xx_out[(long long)t * a.xx_stride + d] = __float2half_rn(xx[i]);
        for (int m = 0; m < a.n_mix; ++m) {
            const float mv = __half2float(a.mix[m][(long long)t * a.mix_stride + d]);
            float o;
            if (a.mode == 0) o = r16(r16(xx[i] * mv) + r16(prev[i] * r16(1.0f - mv)));
            else o = r16(xx[i] + r16(r16(prev[i] - xx[i]) * mv));
            a.out[m][(long long)t * a.out_stride + d] = __float2half_rn(o);
        }
        if (t == a.T - 1 && a.new_state) a.new_state[d] = __float2half_rn(xx[i]);
    }
}

// The same computation with 16-byte accesses, every load of a row issued before the first reduction: the form for
// aligned operands (D % 8 == 0, pointers 16-byte aligned, strides multiples of 8).  With a handful of rows (batched
// decode) the per-element form above spends ~30 us in dependent scalar loads from cold memory; this one ~4 us.
template <int VPT>      // vectors of 8 per thread: D <= 2048 * VPT
__global__ void __launch_bounds__(kLnThreads) ln_mix_vec_kernel(const LnMixArgs a) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float sh[kLnThreads / 32];
    const int t = blockIdx.x;
    const int nvec = a.D >> 3;
    const bool own_state = t == 0 || a.sx_stride != 0;      // else the previous row's LayerNorm output is the state
    const bool mixing = a.n_mix > 0;
    uint4 xv[VPT], pv[VPT], wv[VPT], bv[VPT], mv[5][VPT];
    const uint4* xrow = reinterpret_cast<const uint4*>(a.x + (long long)t * a.x_stride);
    const uint4* prow = mixing ? (own_state ? reinterpret_cast<const uint4*>(a.sx + (long long)t * a.sx_stride)
                                            : reinterpret_cast<const uint4*>(a.x + (long long)(t - 1) * a.x_stride)) : nullptr;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * kLnThreads;
        const bool ok = v < nvec;
        xv[i] = ok ? xrow[v] : make_uint4(0, 0, 0, 0);
        pv[i] = (ok && mixing) ? prow[v] : make_uint4(0, 0, 0, 0);
        wv[i] = ok ? reinterpret_cast<const uint4*>(a.ln_w)[v] : make_uint4(0, 0, 0, 0);
        bv[i] = ok ? reinterpret_cast<const uint4*>(a.ln_b)[v] : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int m = 0; m < 5; ++m)
            mv[m][i] = (ok && m < a.n_mix) ? reinterpret_cast<const uint4*>(a.mix[m] + (long long)t * a.mix_stride)[v] : make_uint4(0, 0, 0, 0);
    }
    // statistics of this row and, in sequence mode, of the previous one (two passes each, as layer_norm_row)
    auto stats = [&](const uint4 (&r)[VPT], float& mean, float& rstd) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const __half2* h = reinterpret_cast<const __half2*>(&r[i]);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h[e]); s += f.x; s += f.y; }
        }
        mean = block_sum(s, sh) / float(a.D);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            if (threadIdx.x + i * kLnThreads < nvec) {
                const __half2* h = reinterpret_cast<const __half2*>(&r[i]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h[e]);
                    q = fmaf(f.x - mean, f.x - mean, q);
                    q = fmaf(f.y - mean, f.y - mean, q);
                }
            }
        }
        rstd = rsqrtf(block_sum(q, sh) / float(a.D) + 1e-5f);
    };
    float mean, rstd, pmean = 0.f, prstd = 0.f;
    stats(xv, mean, rstd);
    if (mixing && !own_state) stats(pv, pmean, prstd);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * kLnThreads;
        if (v >= nvec) continue;
        const __half* hx = reinterpret_cast<const __half*>(&xv[i]);
        const __half* hp = reinterpret_cast<const __half*>(&pv[i]);
        const __half* hw = reinterpret_cast<const __half*>(&wv[i]);
        const __half* hb = reinterpret_cast<const __half*>(&bv[i]);
        float xx[8], prev[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float w = __half2float(hw[e]), b = __half2float(hb[e]);
            xx[e] = r16((__half2float(hx[e]) - mean) * rstd * w + b);
            prev[e] = own_state ? __half2float(hp[e]) : r16((__half2float(hp[e]) - pmean) * prstd * w + b);
        }
        uint4 o;
        __half* ho = reinterpret_cast<__half*>(&o);
        if (a.xx_out || (t == a.T - 1 && a.new_state)) {
#pragma unroll
            for (int e = 0; e < 8; ++e) ho[e] = __float2half_rn(xx[e]);
            if (a.xx_out) reinterpret_cast<uint4*>(a.xx_out + (long long)t * a.xx_stride)[v] = o;
            if (t == a.T - 1 && a.new_state) reinterpret_cast<uint4*>(a.new_state)[v] = o;
        }
#pragma unroll
        for (int m = 0; m < 5; ++m) {
            if (m < a.n_mix) {
                const __half* hm = reinterpret_cast<const __half*>(&mv[m][i]);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float mvv = __half2float(hm[e]);
                    const float r = a.mode == 0 ? r16(r16(xx[e] * mvv) + r16(prev[e] * r16(1.0f - mvv))) : r16(xx[e] + r16(r16(prev[e] - xx[e]) * mvv));
                    ho[e] = __float2half_rn(r);
                }
                reinterpret_cast<uint4*>(a.out[m] + (long long)t * a.out_stride)[v] = o;
            }
        }
    }
}

// RWKV-4 one-step WKV (pkg/model.py:1041-1055): k, v are the fp16 matmul results widened to
// fp32; r already went through sigmoid; out = r * wkv in fp16; state in place.
__global__ void wkv4_one_kernel(int C, const float* __restrict__ t_decay, const float* __restrict__ t_first,
                                const __half* __restrict__ r, const __half* __restrict__ k,
                                const __half* __restrict__ v, float* __restrict__ aa, float* __restrict__ bb,
                                float* __restrict__ pp, __half* __restrict__ out) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float kk = __half2float(k[c]), vv = __half2float(v[c]);
    const float a = aa[c], b = bb[c], p0 = pp[c];
    float ww = t_first[c] + kk;
    float p = fmaxf(p0, ww);
    float e1 = expf(p0 - p), e2 = expf(ww - p);
    const float wkv = r16((e1 * a + e2 * vv) / (e1 * b + e2));
    ww = t_decay[c] + p0;
    p = fmaxf(ww, kk);
    e1 = expf(ww - p); e2 = expf(kk - p);
    aa[c] = e1 * a + e2 * vv;
    bb[c] = e1 * b + e2;
    pp[c] = p;
    out[c] = __float2half_rn(__half2float(r[c]) * wkv);
}

// x = emb[token]: the embedding row of a decode step (model.py:1475), the first node of a token's CUDA graph.  The
// launch that follows starts under it (programmatic dependent launch) and fills its weight ring meanwhile; a library
// gather in this place is a full kernel boundary.  An id outside [0, V) reads row 0 or V - 1 instead of faulting.
__global__ void __launch_bounds__(256) embed_row_kernel(int D, long long V, const __half* __restrict__ emb, long long row_stride,
                                                        const long long* __restrict__ token, __half* __restrict__ out, int vec) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    long long t = *token;
    t = t < 0 ? 0 : (t >= V ? V - 1 : t);
    const __half* row = emb + t * row_stride;
    if (vec) {
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < (D >> 3); i += gridDim.x * blockDim.x)
            reinterpret_cast<uint4*>(out)[i] = __ldg(reinterpret_cast<const uint4*>(row) + i);
    } else {
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < D; i += gridDim.x * blockDim.x) out[i] = row[i];
    }
}

}  // namespace

extern "C" int rwkv_ln_mix(int64_t T, int64_t D, const void* x, int64_t x_stride, const void* sx,
                           const void* ln_w, const void* ln_b, int mode, int n_mix,
                           const void* const* mix, int64_t mix_stride, void* const* out, int64_t out_stride,
                           void* xx_out, int64_t xx_stride, void* new_state, void* stream) {
    return rwkv_ln_mix_rows(T, D, x, x_stride, sx, 0, ln_w, ln_b, mode, n_mix, mix, mix_stride, out, out_stride, xx_out, xx_stride,
                            new_state, stream);
}

extern "C" int rwkv_ln_mix_rows(int64_t T, int64_t D, const void* x, int64_t x_stride, const void* sx, int64_t sx_stride,
                                const void* ln_w, const void* ln_b, int mode, int n_mix,
                                const void* const* mix, int64_t mix_stride, void* const* out, int64_t out_stride,
                                void* xx_out, int64_t xx_stride, void* new_state, void* stream) {
    RWKV_CHECK_ARG(T >= 1 && T <= INT32_MAX && D >= 1 && D <= kLnThreads * kLnMaxPer);
    RWKV_CHECK_ARG(x && ln_w && ln_b && n_mix >= 0 && n_mix <= 5 && (mode == 0 || mode == 1));
    RWKV_CHECK_ARG(n_mix == 0 || (sx && mix && out));
    LnMixArgs a;
    a.x = (const __half*)x; a.x_stride = x_stride; a.sx = (const __half*)sx; a.sx_stride = sx_stride;
    a.ln_w = (const __half*)ln_w; a.ln_b = (const __half*)ln_b;
    for (int m = 0; m < 5; ++m) {
        a.mix[m] = m < n_mix ? (const __half*)mix[m] : nullptr;
        a.out[m] = m < n_mix ? (__half*)out[m] : nullptr;
        RWKV_CHECK_ARG(m >= n_mix || (a.mix[m] && a.out[m]));
    }
    a.mix_stride = mix_stride; a.out_stride = out_stride;
    a.xx_out = (__half*)xx_out; a.xx_stride = xx_stride; a.new_state = (__half*)new_state;
    a.T = int(T); a.D = int(D); a.n_mix = n_mix; a.mode = mode;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // aligned operands: the 16-byte form
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    bool vec = D % 8 == 0 && al16(x) && x_stride % 8 == 0 && al16(ln_w) && al16(ln_b) && mix_stride % 8 == 0 && out_stride % 8 == 0 &&
               (xx_out == nullptr || (al16(xx_out) && xx_stride % 8 == 0)) && (new_state == nullptr || al16(new_state)) &&
               (n_mix == 0 || (al16(sx) && sx_stride % 8 == 0));
    for (int m = 0; m < n_mix; ++m) vec = vec && al16(mix[m]) && al16(out[m]);
    static int use_vec = -1;
    if (use_vec < 0) { const char* e = getenv("RWKV_B200_LN_VEC"); use_vec = (e != nullptr && e[0] == '0') ? 0 : 1; }
    if (vec && use_vec) {
        const int vpt = int((D / 8 + kLnThreads - 1) / kLnThreads);
        if (vpt <= 1) return rwkv_launch_pdl(ln_mix_vec_kernel<1>, dim3(int(T)), dim3(kLnThreads), 0, st, a);
        if (vpt <= 2) return rwkv_launch_pdl(ln_mix_vec_kernel<2>, dim3(int(T)), dim3(kLnThreads), 0, st, a);
        return rwkv_launch_pdl(ln_mix_vec_kernel<4>, dim3(int(T)), dim3(kLnThreads), 0, st, a);
    }
    const int per = int((D + kLnThreads - 1) / kLnThreads);
    if (per <= 4) return rwkv_launch_pdl(ln_mix_kernel<4>, dim3(int(T)), dim3(kLnThreads), 0, st, a);
    if (per <= 16) return rwkv_launch_pdl(ln_mix_kernel<16>, dim3(int(T)), dim3(kLnThreads), 0, st, a);
    return rwkv_launch_pdl(ln_mix_kernel<kLnMaxPer>, dim3(int(T)), dim3(kLnThreads), 0, st, a);
}

extern "C" int rwkv_embed_row(int64_t D, int64_t V, const void* emb, int64_t row_stride, const int64_t* token, void* out,
                              void* stream) {
    RWKV_CHECK_ARG(D >= 1 && D <= INT32_MAX && V >= 1 && row_stride >= D && emb && token && out);
    const int vec = (D % 8 == 0 && row_stride % 8 == 0 && reinterpret_cast<uintptr_t>(emb) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(out) % 16 == 0) ? 1 : 0;
    const int per = vec ? int(D / 8) : int(D);
    return rwkv_launch_pdl(embed_row_kernel, dim3(unsigned(std::min(8, (per + 255) / 256))), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), int(D), (long long)V, static_cast<const __half*>(emb),
                           (long long)row_stride, reinterpret_cast<const long long*>(token), static_cast<__half*>(out), vec);
}

extern "C" int rwkv_wkv4_one(int64_t C, const float* t_decay, const float* t_first, const void* r,
                             const void* k, const void* v, float* aa, float* bb, float* pp, void* out,
                             void* stream) {
    RWKV_CHECK_ARG(C >= 1 && C <= INT32_MAX && t_decay && t_first && r && k && v && aa && bb && pp && out);
    return rwkv_launch_pdl(wkv4_one_kernel, dim3(int((C + 127) / 128)), dim3(128), 0,
                           static_cast<cudaStream_t>(stream), int(C), t_decay, t_first, (const __half*)r,
                           (const __half*)k, (const __half*)v, aa, bb, pp, (__half*)out);
}
