// The decode step as ONE persistent kernel over a re-tiled copy of the packed weights ("weight
// stream").
//
// A token of RWKV is a chain of dependent matrix-vector products (four per RWKV-4 layer: r/k/v,
// output, ffn r/k, ffn value; pkg/model.py:984-992, 1034-1055), each of which has to stream its
// uint8 matrix from HBM once.  Launch by launch, the HBM idles at every dependency: the next
// launch's CTAs cannot prefetch before they are resident.  Here one CTA per SM lives for the whole
// token and the weights are laid out for it:
//
//   * Every matrix is split by OUTPUT columns over the CTAs (units of 4 columns), so a CTA owns
//     whole dot products: no split-K, no cross-CTA reduction, results are exact integer sums.
//   * The bytes a CTA needs, for all matrices of the token in the order it needs them, are ONE
//     contiguous region of the stream buffer, already in the order its threads consume them
//     (8-byte cells = 2 rows x 4 columns with the rows interleaved for dp2a).  A producer warp
//     copies it through a ring of 16 KB shared-memory slots with cp.async.bulk + mbarrier,
//     running ahead of the math across matrix and phase boundaries: while the CTAs exchange a
//     result vector, HBM keeps filling the rings (up to ~150 KB per SM).
//   * Between dependent matrices ("phases") the CTAs meet at a grid barrier (one atomic counter,
//     bounded spin), read the full input vector from L2 and redo the cheap pointwise prologue
//     (LayerNorm + token-shift mix, RWKV-4 WKV step) redundantly.
//
// Arithmetic: x' = x * ry is quantised per vector to 30-bit fixed point (q = hi * 2^15 + lo),
// both halves go through dp2a against the raw codes, sums are kept in 64-bit integers: the
// streamed part of mm8_one (operators.cu:224-230) is computed exactly for the quantised x', whose
// relative error (2^-24 of fp32 for large entries, 2^-30 of the largest entry for small ones) is
// that of an fp32 product.  Results do not depend on any summation order.
#include "common.cuh"

namespace {

constexpr int kConsumers = 512;
constexpr int kConsWarps = kConsumers / 32;
constexpr int kStreamThreads = kConsumers + 32;          // + the producer warp
constexpr int kIter = 4;                                 // cells per thread and stage
constexpr int kSlotBytes = kIter * kConsumers * 8;       // 16 KB
constexpr int kRedBytes = 128 * 4 * 8;                   // [<= 128 subgroups][4 columns] 64-bit sums
constexpr int kMaxSlots = 12;
constexpr int kMaxCtas = 160;
constexpr int kMaxPhaseProblems = 4;
constexpr int kFlushStages = 16;                         // 32-bit partial sums are widened every 16 stages
constexpr float kQMax = 1.0e9f;                          // |q| <= 1e9 < 2^30: hi fits 16 signed bits with margin
constexpr unsigned long long kWaitNs = 2000000000ull;    // every wait gives up after 2 s

struct SProblem {
    const void* x;
    const void* mx;
    const void* rx;
    const void* my;
    const void* ry;
    void* y;
    const void* aux;
    const void* aux2;
    int N, M, epilogue, prologue, mode;
    float out_scale;
    // RWKV_PRO_LN_MIX: p0 ln weight, p1 ln bias, p2 previous token's LayerNorm output, p3 mix, q0 LayerNorm out
    // RWKV_PRO_WKV4:   p0 k, p1 v; f0 t_decay, f1 t_first, f2..f4 aa, bb, pp in; g0..g2 aa, bb, pp out
    const void *p0, *p1, *p2, *p3;
    void* q0;
    const float *f0, *f1, *f2, *f3, *f4;
    float *g0, *g1, *g2;
    int xq_off;         // byte offset of this problem's activations in shared memory
    int share_ln;       // same x and LayerNorm as the previous problem of the phase: statistics reused
};

struct SPhase {
    int count;
    int pad;
    SProblem p[kMaxPhaseProblems];
};

struct STable {
    int n_phases, n_ctas, xq_bytes, n_slots;
    long long cta_base[kMaxCtas];       // byte offset of every CTA's region in the weight stream
    // SPhase phases[n_phases] follow
};

// How one matrix is laid out for one CTA.
struct Geom {
    int Q;              // column quads owned by this CTA (4 columns each)
    int u0;             // first quad
    int SG;             // lanes that share a quad inside a warp (4, 8, 16 or 32)
    int PPI;            // row pairs per iteration (= SG * subgroups per quad)
    int TA;             // active threads = Q * PPI
    int kp;             // row pairs, rounded up to a multiple of SG
    int cells;          // kp * Q
    int n_stages;
    long long bytes;    // cells * 8
};

__host__ __device__ inline Geom seg_geom(int N, int M, int cta, int G) {
    Geom g;
    const int U = (M + 3) >> 2;
    const int base = U / G, rem = U % G;
    g.Q = base + (cta < rem ? 1 : 0);
    g.u0 = cta * base + (cta < rem ? cta : rem);
    g.SG = 4; g.PPI = 0; g.TA = 0; g.kp = 0; g.cells = 0; g.n_stages = 0; g.bytes = 0;
    if (g.Q == 0 || g.Q > kConsumers / 4) return g;       // more than 128 quads per CTA: not planned (see plan)
    int best_ta = 0;
    for (int sg = 32; sg >= 4; sg >>= 1) {
        const int nsub = (kConsumers / sg) / g.Q;
        const int ta = nsub * g.Q * sg;
        if (ta > best_ta) { best_ta = ta; g.SG = sg; }
    }
    g.TA = best_ta;
    g.PPI = best_ta / g.Q;
    const int kp = (N + 1) >> 1;
    g.kp = (kp + g.SG - 1) / g.SG * g.SG;
    g.cells = g.kp * g.Q;
    const int per_stage = kIter * g.TA;
    g.n_stages = (g.cells + per_stage - 1) / per_stage;
    g.bytes = (long long)g.cells * 8;
    return g;
}

// ---------------------------------------------------------------------------------------------
// PTX helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t s2u(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"((uint64_t)__cvta_generic_to_global(src)), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }
__device__ __forceinline__ int dp2a_lo(int a, uint32_t b, int c) {
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi(int a, uint32_t b, int c) {
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Bounded wait on an mbarrier phase.  After the first give-up in this CTA (*err set) later waits
// poll only a few times, so a broken pipeline drains quickly instead of timing out stage by stage.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* err, unsigned* gerr) {
    if (mbar_try(bar, parity)) return;
    const unsigned long long t0 = gtime();
    for (unsigned it = 0;; ++it) {
        if (mbar_try(bar, parity)) return;
        if (*err != 0 && it > 4) return;
        if ((it & 255) == 255 && gtime() - t0 > kWaitNs) {
            *err = 1;
            atomicExch(gerr, 1u);
            return;
        }
    }
}

struct SharedCtl {
    unsigned long long full[kMaxSlots];
    unsigned long long empty[kMaxSlots];
    float wsum[kMaxPhaseProblems][kConsWarps][3];     // per warp: sum x, sum x', sum x*my
    int wsumi[kMaxPhaseProblems][kConsWarps][2];      // per warp: sum hi, sum lo
    float inv_scale[kMaxPhaseProblems];
    float red16[kConsWarps];
    int err;
};

__device__ __forceinline__ float cons_block_sum(float v, float* sh, int warp, int lane) {
    v = warp_sum(v);
    cons_sync();
    if (lane == 0) sh[warp] = v;
    cons_sync();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kConsWarps; ++i) t += sh[i];
    return t;
}
__device__ __forceinline__ float cons_block_max(float v, float* sh, int warp, int lane) {
    v = warp_max(v);
    cons_sync();
    if (lane == 0) sh[warp] = v;
    cons_sync();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kConsWarps; ++i) t = fmaxf(t, sh[i]);
    return t;
}

__device__ __forceinline__ void h8_to_f(const uint4& v, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float2 t = __half22float2(h[e]); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
}
__device__ __forceinline__ uint4 f_to_h8(const float (&f)[8]) {
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(f[2 * e], f[2 * e + 1]);
    return v;
}
__device__ __forceinline__ uint4 ldcg16(const void* base, int j8) { return __ldcg(reinterpret_cast<const uint4*>(base) + (j8 >> 3)); }
__device__ __forceinline__ uint4 ldg16(const void* base, int j8) { return __ldg(reinterpret_cast<const uint4*>(base) + (j8 >> 3)); }

// The W (4 or 8) activations starting at element j are multiplied with ry, written as fp32 x' and
// added to the running sums.  A NaN anywhere makes the maximum infinite (a NaN does not survive fmaxf).
template <int W>
__device__ __forceinline__ void emit(const float (&xv)[W], const SProblem& P, int j, float* xs, float& sx, float& sxr,
                                     float& sxmy, float& xmax) {
    float ry[W], my[W];
    if (W == 8) {
        float a[8], b[8];
        h8_to_f(ldg16(P.ry, j), a);
        h8_to_f(ldg16(P.my, j), b);
#pragma unroll
        for (int e = 0; e < W; ++e) { ry[e] = a[e]; my[e] = b[e]; }
    } else {
        const uint2 a = __ldg(reinterpret_cast<const uint2*>(static_cast<const __half*>(P.ry) + j));
        const uint2 b = __ldg(reinterpret_cast<const uint2*>(static_cast<const __half*>(P.my) + j));
        const __half2* ha = reinterpret_cast<const __half2*>(&a);
        const __half2* hb = reinterpret_cast<const __half2*>(&b);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const float2 fa = __half22float2(ha[e]), fb = __half22float2(hb[e]);
            ry[2 * e] = fa.x; ry[2 * e + 1] = fa.y; my[2 * e] = fb.x; my[2 * e + 1] = fb.y;
        }
    }
    float xp[W];
#pragma unroll
    for (int e = 0; e < W; ++e) {
        xp[e] = xv[e] * ry[e];
        sx += xv[e];
        sxr += xp[e];
        sxmy = fmaf(xv[e], my[e], sxmy);
        xmax = (xp[e] == xp[e]) ? fmaxf(xmax, fabsf(xp[e])) : __int_as_float(0x7f800000);
    }
#pragma unroll
    for (int e = 0; e < W; e += 4) *reinterpret_cast<float4*>(xs + j + e) = make_float4(xp[e], xp[e + 1], xp[e + 2], xp[e + 3]);
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kStreamThreads, 1)
mm8_stream_kernel(const STable* __restrict__ table, const uint8_t* __restrict__ wstream, unsigned* sync_words,
                  unsigned long long* trace) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, G = gridDim.x;
    const int n_phases = table->n_phases, n_slots = table->n_slots, xq_bytes = table->xq_bytes;
    const SPhase* phases = reinterpret_cast<const SPhase*>(table + 1);
    uint8_t* xq_base = smem;
    long long* red = reinterpret_cast<long long*>(smem + xq_bytes);
    uint8_t* ring = smem + xq_bytes + kRedBytes;
    SharedCtl* ctl = reinterpret_cast<SharedCtl*>(ring + (size_t)n_slots * kSlotBytes);
    unsigned* gbar = sync_words;            // grid barrier counter (zeroed by the host before the launch)
    unsigned* gerr = sync_words + 1;        // error word

    if (tid == 0) {
        for (int s = 0; s < n_slots; ++s) {
            mbar_init(s2u(&ctl->full[s]), 1);
            mbar_init(s2u(&ctl->empty[s]), kConsWarps);
        }
        ctl->err = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    volatile int* err = &ctl->err;

    if (warp == kConsWarps) {
        // ================= producer: one thread walks this CTA's region of the stream =================
        if (lane == 0) {
            const uint8_t* src = wstream + table->cta_base[cta];
            int slot = 0;
            uint32_t parity = 1;            // a fresh mbarrier passes a wait on parity 1: every slot starts empty
            for (int ph = 0; ph < n_phases; ++ph) {
                const int count = phases[ph].count;
                for (int z = 0; z < count; ++z) {
                    const Geom g = seg_geom(phases[ph].p[z].N, phases[ph].p[z].M, cta, G);
                    const long long stage_bytes = (long long)kIter * g.TA * 8;
                    for (int s = 0; s < g.n_stages; ++s) {
                        const long long left = g.bytes - s * stage_bytes;
                        const uint32_t bytes = (uint32_t)(left < stage_bytes ? left : stage_bytes);
                        mbar_wait(s2u(&ctl->empty[slot]), parity, err, gerr);
                        mbar_expect_tx(s2u(&ctl->full[slot]), bytes);
                        bulk_g2s(s2u(ring + (size_t)slot * kSlotBytes), src + s * stage_bytes, bytes, s2u(&ctl->full[slot]));
                        if (++slot == n_slots) { slot = 0; parity ^= 1; }
                    }
                    src += g.bytes;
                }
            }
        }
        return;
    }

    // ================= consumers =================
    int slot = 0;
    uint32_t parity = 0;
    for (int ph = 0; ph < n_phases; ++ph) {
        const SPhase& PH = phases[ph];
        const int count = PH.count;

        // ---- prologue: every CTA builds the full quantised activation vector of each problem ----
        uint4 lnx[2];
        float mean = 0.f, rstd = 0.f;
        lnx[0] = lnx[1] = make_uint4(0, 0, 0, 0);
        for (int z = 0; z < count; ++z) {
            const SProblem& P = PH.p[z];
            const int N = P.N;
            float* xs = reinterpret_cast<float*>(xq_base + P.xq_off);
            float sx = 0.f, sxr = 0.f, sxmy = 0.f, xmax = 0.f;
            if (P.prologue == RWKV_PRO_LN_MIX) {
                if (!P.share_ln) {          // statistics of the residual stream (N <= 8192: two 16-byte loads per thread)
                    float s = 0.f;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int j8 = (tid + i * kConsumers) * 8;
                        lnx[i] = j8 < N ? ldcg16(P.x, j8) : make_uint4(0, 0, 0, 0);
                        float f[8];
                        h8_to_f(lnx[i], f);
#pragma unroll
                        for (int e = 0; e < 8; ++e) s += f[e];
                    }
                    mean = cons_block_sum(s, ctl->red16, warp, lane) / float(N);
                    float q = 0.f;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        if ((tid + i * kConsumers) * 8 < N) {
                            float f[8];
                            h8_to_f(lnx[i], f);
#pragma unroll
                            for (int e = 0; e < 8; ++e) q = fmaf(f[e] - mean, f[e] - mean, q);
                        }
                    }
                    rstd = rsqrtf(cons_block_sum(q, ctl->red16, warp, lane) / float(N) + 1e-5f);
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int j8 = (tid + i * kConsumers) * 8;
                    if (j8 < N) {
                        float f[8], lw[8], lb[8], xv[8];
                        h8_to_f(lnx[i], f);
                        h8_to_f(ldg16(P.p0, j8), lw);
                        h8_to_f(ldg16(P.p1, j8), lb);
#pragma unroll
                        for (int e = 0; e < 8; ++e) xv[e] = r16((f[e] - mean) * rstd * lw[e] + lb[e]);
                        if (P.q0 != nullptr && ((j8 >> 3) % G) == cta)
                            *reinterpret_cast<uint4*>(static_cast<__half*>(P.q0) + j8) = f_to_h8(xv);
                        if (P.mode != 2) {
                            float sv[8], mv[8];
                            h8_to_f(ldcg16(P.p2, j8), sv);
                            h8_to_f(ldg16(P.p3, j8), mv);
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                xv[e] = P.mode == 0 ? r16(r16(xv[e] * mv[e]) + r16(sv[e] * r16(1.0f - mv[e])))
                                                    : r16(xv[e] + r16(r16(sv[e] - xv[e]) * mv[e]));
                        }
                        emit<8>(xv, P, j8, xs, sx, sxr, sxmy, xmax);
                    }
                }
            } else if (P.prologue == RWKV_PRO_WKV4) {       // pkg/model.py:1041-1055, four channels per thread and pass
                for (int j = tid * 4; j < N; j += kConsumers * 4) {
                    const uint2 r2 = __ldcg(reinterpret_cast<const uint2*>(static_cast<const __half*>(P.x) + j));
                    const uint2 k2 = __ldcg(reinterpret_cast<const uint2*>(static_cast<const __half*>(P.p0) + j));
                    const uint2 v2 = __ldcg(reinterpret_cast<const uint2*>(static_cast<const __half*>(P.p1) + j));
                    const float4 a4 = __ldcg(reinterpret_cast<const float4*>(P.f2 + j));
                    const float4 b4 = __ldcg(reinterpret_cast<const float4*>(P.f3 + j));
                    const float4 p4 = __ldcg(reinterpret_cast<const float4*>(P.f4 + j));
                    const float4 d4 = __ldg(reinterpret_cast<const float4*>(P.f0 + j));
                    const float4 f4 = __ldg(reinterpret_cast<const float4*>(P.f1 + j));
                    const float aa[4] = {a4.x, a4.y, a4.z, a4.w}, bb[4] = {b4.x, b4.y, b4.z, b4.w}, pp[4] = {p4.x, p4.y, p4.z, p4.w};
                    const float td[4] = {d4.x, d4.y, d4.z, d4.w}, tf[4] = {f4.x, f4.y, f4.z, f4.w};
                    const __half* rh = reinterpret_cast<const __half*>(&r2);
                    const __half* kh = reinterpret_cast<const __half*>(&k2);
                    const __half* vh = reinterpret_cast<const __half*>(&v2);
                    float xv[4], na[4], nb[4], np[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float kk = __half2float(kh[e]), vv = __half2float(vh[e]);
                        float ww = tf[e] + kk;
                        float p = fmaxf(pp[e], ww);
                        float e1 = expf(pp[e] - p), e2 = expf(ww - p);
                        const float wkv = r16((e1 * aa[e] + e2 * vv) / (e1 * bb[e] + e2));
                        ww = td[e] + pp[e];
                        p = fmaxf(ww, kk);
                        e1 = expf(ww - p); e2 = expf(kk - p);
                        na[e] = e1 * aa[e] + e2 * vv;
                        nb[e] = e1 * bb[e] + e2;
                        np[e] = p;
                        xv[e] = r16(__half2float(rh[e]) * wkv);
                    }
                    if (((j >> 3) % G) == cta) {
                        *reinterpret_cast<float4*>(P.g0 + j) = make_float4(na[0], na[1], na[2], na[3]);
                        *reinterpret_cast<float4*>(P.g1 + j) = make_float4(nb[0], nb[1], nb[2], nb[3]);
                        *reinterpret_cast<float4*>(P.g2 + j) = make_float4(np[0], np[1], np[2], np[3]);
                    }
                    emit<4>(xv, P, j, xs, sx, sxr, sxmy, xmax);
                }
            } else {
                for (int j8 = tid * 8; j8 < N; j8 += kConsumers * 8) {
                    float xv[8];
                    h8_to_f(ldcg16(P.x, j8), xv);
                    emit<8>(xv, P, j8, xs, sx, sxr, sxmy, xmax);
                }
            }
            sx = warp_sum(sx); sxr = warp_sum(sxr); sxmy = warp_sum(sxmy);
            if (lane == 0) { ctl->wsum[z][warp][0] = sx; ctl->wsum[z][warp][1] = sxr; ctl->wsum[z][warp][2] = sxmy; }
            const float m = cons_block_max(xmax, ctl->red16, warp, lane);     // also orders the x' stores before the reads below
            const bool finite = m < 3.0e38f;
            const float scale = (finite && m > 0.f) ? kQMax / m : 0.f;
            if (tid == 0) ctl->inv_scale[z] = !finite ? __int_as_float(0x7fc00000) : (m > 0.f ? m / kQMax : 0.f);
            // quantise in place: pair p (rows 2p, 2p+1) becomes {hi(2p) | hi(2p+1) << 16, lo(2p) | lo(2p+1) << 16}
            const int kp32 = (((N + 1) >> 1) + 31) & ~31;
            int shi = 0, slo = 0;
            for (int p = tid; p < kp32; p += kConsumers) {
                const int j = 2 * p;
                const float2 v = *reinterpret_cast<const float2*>(xs + j);
                const int q0 = j < N ? __float2int_rn(v.x * scale) : 0;
                const int q1 = j + 1 < N ? __float2int_rn(v.y * scale) : 0;
                const int h0 = q0 >> 15, h1 = q1 >> 15, l0 = q0 & 0x7fff, l1 = q1 & 0x7fff;
                shi += h0 + h1;
                slo += l0 + l1;
                *reinterpret_cast<uint2*>(xs + j) = make_uint2((uint32_t(h0) & 0xffffu) | (uint32_t(h1) << 16),
                                                               uint32_t(l0) | (uint32_t(l1) << 16));
            }
            shi = warp_sum_i(shi); slo = warp_sum_i(slo);
            if (lane == 0) { ctl->wsumi[z][warp][0] = shi; ctl->wsumi[z][warp][1] = slo; }
        }
        cons_sync();
        if (trace != nullptr && tid == 0 && cta < 2) trace[(ph * 2 + cta) * 4 + 2] = gtime();

        // ---- the matrices of the phase, one after the other ----
        for (int z = 0; z < count; ++z) {
            const SProblem& P = PH.p[z];
            const Geom g = seg_geom(P.N, P.M, cta, G);
            const uint2* xq = reinterpret_cast<const uint2*>(xq_base + P.xq_off);
            const int sub = tid / g.SG, lane_in = tid % g.SG;
            const bool active = tid < g.TA;
            const int gg = active ? (sub / g.Q) * g.SG + lane_in : 0;      // this thread's row pair within an iteration
            int ah[4] = {0, 0, 0, 0}, al[4] = {0, 0, 0, 0};
            long long th[4] = {0, 0, 0, 0}, tl[4] = {0, 0, 0, 0};
            int since = 0;
            for (int s = 0; s < g.n_stages; ++s) {
                mbar_wait(s2u(&ctl->full[slot]), parity, err, gerr);
                const uint8_t* sp = ring + (size_t)slot * kSlotBytes;
                uint2 w[kIter], xv[kIter];
#pragma unroll
                for (int r = 0; r < kIter; ++r) {
                    const int it = s * kIter + r;
                    const bool ok = active && it * g.TA + tid < g.cells;
                    w[r] = ok ? *reinterpret_cast<const uint2*>(sp + (size_t)(r * g.TA + tid) * 8) : make_uint2(0, 0);
                    xv[r] = ok ? xq[it * g.PPI + gg] : make_uint2(0, 0);
                }
#pragma unroll
                for (int r = 0; r < kIter; ++r) {
                    ah[0] = dp2a_lo((int)xv[r].x, w[r].x, ah[0]);
                    ah[1] = dp2a_hi((int)xv[r].x, w[r].x, ah[1]);
                    ah[2] = dp2a_lo((int)xv[r].x, w[r].y, ah[2]);
                    ah[3] = dp2a_hi((int)xv[r].x, w[r].y, ah[3]);
                    al[0] = dp2a_lo((int)xv[r].y, w[r].x, al[0]);
                    al[1] = dp2a_hi((int)xv[r].y, w[r].x, al[1]);
                    al[2] = dp2a_lo((int)xv[r].y, w[r].y, al[2]);
                    al[3] = dp2a_hi((int)xv[r].y, w[r].y, al[3]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(s2u(&ctl->empty[slot]));
                if (++slot == n_slots) { slot = 0; parity ^= 1; }
                if (++since == kFlushStages) {
                    since = 0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) { th[i] += ah[i]; tl[i] += al[i]; ah[i] = 0; al[i] = 0; }
                }
            }
            // this thread's exact sums of q * w for its four columns; add the lanes of the subgroup
            long long S[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) S[i] = ((th[i] + ah[i]) << 15) + (tl[i] + al[i]);
            for (int o = g.SG >> 1; o > 0; o >>= 1) {
#pragma unroll
                for (int i = 0; i < 4; ++i) S[i] += __shfl_xor_sync(0xffffffffu, S[i], o);
            }
            cons_sync();                    // the previous matrix's partial sums have been read
            if (active && lane_in == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) red[sub * 4 + i] = S[i];
            }
            cons_sync();
            const int nrep = g.Q > 0 ? g.PPI / g.SG : 0;
            for (int kk = tid; kk < 4 * g.Q; kk += kConsumers) {
                const int k = (g.u0 << 2) + kk;
                if (k >= P.M) continue;
                const int qq = kk >> 2, i = kk & 3;
                long long tot = 0;
                for (int rep = 0; rep < nrep; ++rep) tot += red[(rep * g.Q + qq) * 4 + i];
                float tx = 0.f, txr = 0.f, txmy = 0.f;
                long long sq_hi = 0, sq_lo = 0;
#pragma unroll
                for (int w8 = 0; w8 < kConsWarps; ++w8) {
                    tx += ctl->wsum[z][w8][0]; txr += ctl->wsum[z][w8][1]; txmy += ctl->wsum[z][w8][2];
                    sq_hi += ctl->wsumi[z][w8][0]; sq_lo += ctl->wsumi[z][w8][1];
                }
                tot -= 128ll * ((sq_hi << 15) + sq_lo);
                const float sdot = __ll2float_rn(tot) * ctl->inv_scale[z];
                const float rxk = __half2float(__ldg(static_cast<const __half*>(P.rx) + k));
                const float mxk = __half2float(__ldg(static_cast<const __half*>(P.mx) + k));
                const float val = fmaf(rxk, sdot, fmaf(rxk * 128.5f, txr, fmaf(mxk, tx, txmy)));
                __half* yh = static_cast<__half*>(P.y);
                switch (P.epilogue) {
                case RWKV_EPI_ACC_F32: {
                    float* y = static_cast<float*>(P.y);
                    y[k] = __ldcg(y + k) + val;
                    break;
                }
                case RWKV_EPI_STORE: yh[k] = __float2half_rn(val); break;
                case RWKV_EPI_SIGMOID: yh[k] = __float2half_rn(1.0f / (1.0f + expf(-r16(val)))); break;
                case RWKV_EPI_RELU_SQ: { const float v = fmaxf(r16(val), 0.0f); yh[k] = __float2half_rn(v * v); break; }
                case RWKV_EPI_RESIDUAL: {
                    const float a = __half2float(__ldcg(static_cast<const __half*>(P.aux) + k));
                    yh[k] = __float2half_rn(r16(a + r16(val)) * P.out_scale);
                    break;
                }
                case RWKV_EPI_MUL_RESIDUAL: {
                    const float a = __half2float(__ldcg(static_cast<const __half*>(P.aux) + k));
                    const float a2 = __half2float(__ldcg(static_cast<const __half*>(P.aux2) + k));
                    yh[k] = __float2half_rn(r16(a + r16(a2 * r16(val))) * P.out_scale);
                    break;
                }
                case RWKV_EPI_STORE_F32: static_cast<float*>(P.y)[k] = r16(val); break;
                case RWKV_EPI_SILU: { const float v = r16(val); yh[k] = __float2half_rn(v / (1.0f + expf(-v))); break; }
                default: break;
                }
            }
        }
        if (trace != nullptr && tid == 0 && cta < 2) trace[(ph * 2 + cta) * 4 + 3] = gtime();

        // ---- grid barrier: the phase's results are complete and visible before anyone reads them ----
        if (ph + 1 < n_phases) {
            cons_sync();
            if (tid == 0) {
                __threadfence();
                atomicAdd(gbar, 1u);
                if (trace != nullptr && cta < 2) trace[(ph * 2 + cta) * 4 + 0] = gtime();
                const unsigned target = unsigned(G) * unsigned(ph + 1);
                const unsigned long long t0 = gtime();
                for (unsigned it = 0;; ++it) {
                    unsigned v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(gbar) : "memory");
                    if (v >= target || *err != 0) break;
                    if ((it & 63) == 63 && gtime() - t0 > kWaitNs) {
                        *err = 1;
                        atomicExch(gerr, 1u);
                        break;
                    }
                }
                if (trace != nullptr && cta < 2) trace[(ph * 2 + cta) * 4 + 1] = gtime();
            }
            cons_sync();
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Re-tiling: codes of one matrix -> the cells of every CTA's region.
// ---------------------------------------------------------------------------------------------
struct PackArgs {
    const uint8_t* w;
    long long w_stride;
    int N, M, G;
    long long off[kMaxCtas];        // where this matrix's segment starts in the stream, per CTA
};

__global__ void mm8_stream_pack_kernel(PackArgs a, uint8_t* wstream) {
    const int cta = blockIdx.y;
    const Geom g = seg_geom(a.N, a.M, cta, a.G);
    uint2* dst = reinterpret_cast<uint2*>(wstream + a.off[cta]);
    for (int cell = blockIdx.x * blockDim.x + threadIdx.x; cell < g.cells; cell += gridDim.x * blockDim.x) {
        const int it = cell / g.TA, t = cell - it * g.TA;
        const int sub = t / g.SG, lane_in = t % g.SG;
        const int q = sub % g.Q, gg = (sub / g.Q) * g.SG + lane_in;
        const int p = it * g.PPI + gg;
        const int r0 = 2 * p, c0 = (g.u0 + q) * 4;
        uint32_t b[8];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int row = r0 + r, col = c0 + c;
                b[c * 2 + r] = (row < a.N && col < a.M) ? a.w[(long long)row * a.w_stride + col] : 0u;
            }
        }
        dst[cell] = make_uint2(b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24), b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24));
    }
}

int stream_ctas() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        cudaGetLastError();
        return 148;
    }
    return sms > kMaxCtas ? kMaxCtas : sms;
}

bool stream_supported(const rwkv_mm8_problem& q, int G) {
    if (q.N < 8 || q.N % 8 != 0 || q.M < 1) return false;
    if (((q.M + 3) / 4 + G - 1) / G > kConsumers / 4) return false;
    if (q.prologue == RWKV_PRO_LN_MIX && q.N > 2 * kConsumers * 8) return false;
    return true;
}

}  // namespace

extern "C" int rwkv_mm8_stream_ctas(void) { return stream_ctas(); }

extern "C" size_t rwkv_mm8_stream_weight_bytes(const rwkv_mm8_problem* problems, int n_problems, int n_ctas) {
    if (problems == nullptr || n_problems < 1 || n_ctas < 1 || n_ctas > kMaxCtas) return 0;
    size_t total = 0;
    for (int c = 0; c < n_ctas; ++c)
        for (int i = 0; i < n_problems; ++i) total += size_t(seg_geom(problems[i].N, problems[i].M, c, n_ctas).bytes);
    return total + 16;
}

extern "C" int rwkv_mm8_stream_pack(const rwkv_mm8_problem* problems, int n_problems, int n_ctas, void* wstream,
                                    size_t wstream_bytes, void* stream) {
    RWKV_CHECK_ARG(problems != nullptr && n_problems >= 1 && n_ctas >= 1 && n_ctas <= kMaxCtas && wstream != nullptr);
    RWKV_CHECK_ALIGN(wstream, 16);
    if (wstream_bytes < rwkv_mm8_stream_weight_bytes(problems, n_problems, n_ctas)) return RWKV_ERR_WORKSPACE;
    long long base[kMaxCtas], run[kMaxCtas];
    long long total = 0;
    for (int c = 0; c < n_ctas; ++c) {
        base[c] = total;
        run[c] = 0;
        for (int i = 0; i < n_problems; ++i) total += seg_geom(problems[i].N, problems[i].M, c, n_ctas).bytes;
    }
    for (int i = 0; i < n_problems; ++i) {
        const rwkv_mm8_problem& q = problems[i];
        RWKV_CHECK_ARG(q.w != nullptr && q.w_stride >= q.M);
        if (!stream_supported(q, n_ctas)) return RWKV_ERR_UNSUPPORTED;
        PackArgs a;
        a.w = q.w; a.w_stride = q.w_stride; a.N = q.N; a.M = q.M; a.G = n_ctas;
        int max_cells = 0;
        for (int c = 0; c < n_ctas; ++c) {
            const Geom g = seg_geom(q.N, q.M, c, n_ctas);
            a.off[c] = base[c] + run[c];
            run[c] += g.bytes;
            if (g.cells > max_cells) max_cells = g.cells;
        }
        if (max_cells == 0) continue;
        const int bx = (max_cells + 255) / 256 > 64 ? 64 : (max_cells + 255) / 256;
        mm8_stream_pack_kernel<<<dim3(bx, n_ctas), 256, 0, static_cast<cudaStream_t>(stream)>>>(a, static_cast<uint8_t*>(wstream));
        const int rc = rwkv_launch_status();
        if (rc != RWKV_OK) return rc;
    }
    return RWKV_OK;
}

extern "C" size_t rwkv_mm8_stream_table_bytes(int n_phases) {
    return n_phases < 1 ? 0 : sizeof(STable) + size_t(n_phases) * sizeof(SPhase);
}

extern "C" int rwkv_mm8_stream_plan(const rwkv_mm8_problem* problems, const int32_t* counts, int n_phases, int dtype,
                                    int n_ctas, void* table_host, size_t table_bytes) {
    RWKV_CHECK_ARG(problems != nullptr && counts != nullptr && n_phases >= 1 && table_host != nullptr);
    RWKV_CHECK_ARG(n_ctas >= 1 && n_ctas <= kMaxCtas);
    if (dtype != RWKV_F16) return RWKV_ERR_UNSUPPORTED;
    if (table_bytes < rwkv_mm8_stream_table_bytes(n_phases)) return RWKV_ERR_WORKSPACE;
    memset(table_host, 0, rwkv_mm8_stream_table_bytes(n_phases));
    STable* T = static_cast<STable*>(table_host);
    SPhase* PH = reinterpret_cast<SPhase*>(T + 1);
    T->n_phases = n_phases;
    T->n_ctas = n_ctas;
    int xq_max = 0, idx = 0, n_total = 0;
    for (int ph = 0; ph < n_phases; ++ph) {
        RWKV_CHECK_ARG(counts[ph] >= 1 && counts[ph] <= kMaxPhaseProblems);
        PH[ph].count = counts[ph];
        int off = 0;
        for (int z = 0; z < counts[ph]; ++z, ++idx) {
            const rwkv_mm8_problem& q = problems[idx];
            SProblem& P = PH[ph].p[z];
            RWKV_CHECK_ARG(q.x && q.mx && q.rx && q.my && q.ry && q.y);
            RWKV_CHECK_ARG(q.epilogue >= RWKV_EPI_ACC_F32 && q.epilogue <= RWKV_EPI_SILU);
            if (q.epilogue == RWKV_EPI_RESIDUAL || q.epilogue == RWKV_EPI_MUL_RESIDUAL) RWKV_CHECK_ARG(q.aux != nullptr);
            if (q.epilogue == RWKV_EPI_MUL_RESIDUAL) RWKV_CHECK_ARG(q.aux2 != nullptr);
            RWKV_CHECK_ARG(q.prologue >= RWKV_PRO_PLAIN && q.prologue <= RWKV_PRO_WKV4);
            if (!stream_supported(q, n_ctas)) return RWKV_ERR_UNSUPPORTED;
            RWKV_CHECK_ALIGN(q.x, 16); RWKV_CHECK_ALIGN(q.ry, 16); RWKV_CHECK_ALIGN(q.my, 16);
            P.x = q.x; P.mx = q.mx; P.rx = q.rx; P.my = q.my; P.ry = q.ry; P.y = q.y; P.aux = q.aux; P.aux2 = q.aux2;
            P.N = q.N; P.M = q.M; P.epilogue = q.epilogue; P.prologue = q.prologue; P.mode = q.mode; P.out_scale = q.out_scale;
            if (q.prologue == RWKV_PRO_LN_MIX) {
                RWKV_CHECK_ARG(q.ln_w && q.ln_b && q.mode >= 0 && q.mode <= 2);
                if (q.mode != 2) { RWKV_CHECK_ARG(q.sx && q.mix); RWKV_CHECK_ALIGN(q.sx, 16); RWKV_CHECK_ALIGN(q.mix, 16); }
                RWKV_CHECK_ALIGN(q.ln_w, 16); RWKV_CHECK_ALIGN(q.ln_b, 16);
                if (q.xx_out) RWKV_CHECK_ALIGN(q.xx_out, 16);
                P.p0 = q.ln_w; P.p1 = q.ln_b; P.p2 = q.sx; P.p3 = q.mix; P.q0 = q.xx_out;
                P.share_ln = (z > 0 && problems[idx - 1].prologue == RWKV_PRO_LN_MIX && problems[idx - 1].x == q.x &&
                              problems[idx - 1].ln_w == q.ln_w && problems[idx - 1].ln_b == q.ln_b &&
                              problems[idx - 1].N == q.N) ? 1 : 0;
            } else if (q.prologue == RWKV_PRO_WKV4) {
                RWKV_CHECK_ARG(q.k && q.v && q.t_decay && q.t_first && q.aa && q.bb && q.pp && q.aa_out && q.bb_out && q.pp_out);
                RWKV_CHECK_ALIGN(q.k, 16); RWKV_CHECK_ALIGN(q.v, 16); RWKV_CHECK_ALIGN(q.t_decay, 16); RWKV_CHECK_ALIGN(q.t_first, 16);
                RWKV_CHECK_ALIGN(q.aa, 16); RWKV_CHECK_ALIGN(q.bb, 16); RWKV_CHECK_ALIGN(q.pp, 16);
                RWKV_CHECK_ALIGN(q.aa_out, 16); RWKV_CHECK_ALIGN(q.bb_out, 16); RWKV_CHECK_ALIGN(q.pp_out, 16);
                P.p0 = q.k; P.p1 = q.v; P.f0 = q.t_decay; P.f1 = q.t_first; P.f2 = q.aa; P.f3 = q.bb; P.f4 = q.pp;
                P.g0 = q.aa_out; P.g1 = q.bb_out; P.g2 = q.pp_out;
            }
            P.xq_off = off;
            // 4 bytes per row; the row-pair count is padded to 32 so that tails read zeros
            off += ((((q.N + 1) >> 1) + 31) & ~31) * 8;
        }
        if (off > xq_max) xq_max = off;
        n_total += counts[ph];
    }
    T->xq_bytes = (xq_max + 1023) & ~1023;
    int dev = 0, max_smem = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) {
        cudaGetLastError();
        return RWKV_ERR_LAUNCH;
    }
    const int fixed = T->xq_bytes + kRedBytes + int(sizeof(SharedCtl)) + 1024;
    int slots = (max_smem - fixed) / kSlotBytes;
    if (slots > kMaxSlots) slots = kMaxSlots;
    if (slots < 3) return RWKV_ERR_UNSUPPORTED;
    T->n_slots = slots;
    long long total = 0;
    for (int c = 0; c < n_ctas; ++c) {
        T->cta_base[c] = total;
        for (int i = 0; i < n_total; ++i) total += seg_geom(problems[i].N, problems[i].M, c, n_ctas).bytes;
    }
    return RWKV_OK;
}

extern "C" int rwkv_mm8_stream_run(const void* table_dev, const void* table_host, const void* wstream, uint32_t* sync_words,
                                   uint64_t* trace, void* stream) {
    RWKV_CHECK_ARG(table_dev != nullptr && table_host != nullptr && wstream != nullptr && sync_words != nullptr);
    const STable* T = static_cast<const STable*>(table_host);
    const int smem = T->xq_bytes + kRedBytes + T->n_slots * kSlotBytes + int(sizeof(SharedCtl));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaFuncSetAttribute(mm8_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
        cudaMemsetAsync(sync_words, 0, 4, st) != cudaSuccess) {
        cudaGetLastError();
        return RWKV_ERR_LAUNCH;
    }
    const STable* td = static_cast<const STable*>(table_dev);
    const uint8_t* ws = static_cast<const uint8_t*>(wstream);
    unsigned* sw = sync_words;
    unsigned long long* tr = reinterpret_cast<unsigned long long*>(trace);
    void* args[] = {&td, &ws, &sw, &tr};
    // cooperative: all CTAs must be resident at once, they wait for one another at the grid barrier
    if (cudaLaunchCooperativeKernel(reinterpret_cast<void*>(mm8_stream_kernel), dim3(T->n_ctas), dim3(kStreamThreads), args,
                                    size_t(smem), st) != cudaSuccess) {
        cudaGetLastError();
        return RWKV_ERR_LAUNCH;
    }
    return RWKV_OK;
}

// Synchronises `stream`; *error_out = 1 if a wait inside the kernel gave up since the last call
// (the step's results were then undefined), and clears the word.
extern "C" int rwkv_mm8_stream_take_error(uint32_t* sync_words, void* stream, int* error_out) {
    RWKV_CHECK_ARG(sync_words != nullptr && error_out != nullptr);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned v = 0;
    if (cudaMemcpyAsync(&v, sync_words + 1, 4, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess) {
        cudaGetLastError();
        return RWKV_ERR_LAUNCH;
    }
    *error_out = v != 0 ? 1 : 0;
    if (v != 0 && cudaMemsetAsync(sync_words + 1, 0, 4, st) != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    return RWKV_OK;
}
