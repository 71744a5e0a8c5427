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
//     whole dot products: no split-K between CTAs, no cross-CTA reduction, exact integer sums.
//   * The bytes a CTA needs, for all matrices of the token in the order it needs them, are ONE
//     contiguous region of the stream buffer, already in the order its threads consume them
//     (operand fragments of the 8-bit integer tensor-core instruction).  A producer warp copies it
//     through a ring of 16 KB shared-memory slots with cp.async.bulk + mbarrier, running ahead of
//     the math across matrix and phase boundaries: while the CTAs exchange a result vector, HBM
//     keeps filling the rings (~144 KB per SM).
//   * Between dependent matrices ("phases") the CTAs meet at a grid barrier (one atomic counter,
//     bounded spin), read the full input vector from L2 and redo the cheap pointwise prologue
//     (LayerNorm + token-shift mix, RWKV-4 WKV step) redundantly.
//
// Arithmetic: x' = x * ry is quantised per vector to a 31-bit integer q = sum_n d_n 256^n with four
// signed base-256 digits.  mma.sync.m16n8k32.s8.u8 multiplies a 16 x 32 tile whose rows 0..3 are the
// digit planes of 32 consecutive inputs with a 32 x 8 tile of raw codes: D[n][c] = sum_k d_n[k]
// w[k][c] in exact 32-bit integers (|d w| <= 32640, so 65536 inputs cannot overflow).  The streamed
// part of mm8_one (operators.cu:224-230) is therefore computed exactly for the quantised x', whose
// relative error (2^-24 of fp32 for large entries, 2^-30 of the largest entry for small ones) is
// that of an fp32 product; no result depends on a summation order.  The tensor pipe is used because
// it takes one instruction per 256 code bytes where dp2a takes eight: the kernel is HBM-bound and
// the issue slots were what kept the math from catching up after a phase change.
#include "common.cuh"

namespace {

constexpr int kConsumers = 512;
constexpr int kConsWarps = kConsumers / 32;
constexpr int kStreamThreads = kConsumers + 32;          // + the producer warp
constexpr int kSlotBytes = 16384;
constexpr int kMaxOct = 12;                              // column octets a warp accumulates (24 registers)
constexpr int kRedBytes = kConsWarps * kMaxOct * 8 * 8;  // [warp][octet][column] 64-bit partial sums
constexpr int kMaxSlots = 12;
constexpr int kMaxCtas = 160;
constexpr int kMaxPhaseProblems = 4;
constexpr float kQMax = 1.0e9f;                          // |q| <= 1e9 < 2^30
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

// How one matrix is laid out for one CTA.  Its columns are 4 * Q consecutive ones, grouped in
// octets (the N dimension of the instruction; the last octet holds 4 columns when Q is odd); its
// rows in k-blocks of 32 (the K dimension).  One k-block of all the CTA's columns is 128 * Q
// contiguous bytes: per octet 32 (or 16) cells of 8 bytes, cell `lane` = the B fragment of that lane.
// The 16 warps are wo groups along the columns (<= kMaxOct octets each) times wk = 16 / wo along K:
// warp (og, ks) takes the k-blocks kb with kb % wk == ks.
struct Geom {
    int Q;              // column quads owned by this CTA
    int u0;             // first quad
    int n_oct;          // octets, the last one half when Q is odd
    int wo, opw, wk;
    int n_kb;           // ceil(N / 32)
    int kb_bytes;       // 128 * Q
    int kbs;            // k-blocks per stage
    int n_stages;
    long long bytes;
};

__host__ __device__ inline Geom seg_geom(int N, int M, int cta, int G) {
    Geom g;
    const int U = (M + 3) >> 2;
    const int base = U / G, rem = U % G;
    g.Q = base + (cta < rem ? 1 : 0);
    g.u0 = cta * base + (cta < rem ? cta : rem);
    g.n_oct = 0; g.wo = 1; g.opw = 0; g.wk = kConsWarps; g.n_kb = 0; g.kb_bytes = 0; g.kbs = 1; g.n_stages = 0; g.bytes = 0;
    if (g.Q == 0 || g.Q > kSlotBytes / 128) return g;     // more than 128 quads per CTA: not planned (see plan)
    g.n_oct = (g.Q + 1) >> 1;
    while ((g.n_oct + g.wo - 1) / g.wo > kMaxOct) g.wo <<= 1;
    g.opw = (g.n_oct + g.wo - 1) / g.wo;
    g.wk = kConsWarps / g.wo;
    g.n_kb = (N + 31) >> 5;
    g.kb_bytes = 128 * g.Q;
    g.kbs = kSlotBytes / g.kb_bytes;
    if (g.kbs >= g.wk) g.kbs = g.kbs / g.wk * g.wk;       // every K group of warps gets the same share of a stage
    g.n_stages = (g.n_kb + g.kbs - 1) / g.kbs;
    g.bytes = (long long)g.n_kb * g.kb_bytes;
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

// D[16 x 8] (s32) += A[16 x 32] (s8, rows 0..7 in a0 / a2, rows 8..15 zero) * B[32 x 8] (u8).  Only rows
// 0..7 are kept (d0, d1); the other half of the tile multiplies zeros.
__device__ __forceinline__ void imma_16832(int& d0, int& d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    int z0, z1;
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %10, %10};"
                 : "+r"(d0), "+r"(d1), "=r"(z0), "=r"(z1)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "r"(0));
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
    long long wsumq[kMaxPhaseProblems][kConsWarps];   // per warp: sum of the quantised activations
    float wsum[kMaxPhaseProblems][kConsWarps][2];     // per warp: sum x, sum x*my
    float inv_scale[kMaxPhaseProblems];
    float red[kConsWarps][4];
    int err;
};

// Sums (SUM) or maxima of up to four values over the 512 consumer threads.
template <bool SUM>
__device__ __forceinline__ void cons_block_reduce4(float (&v)[4], float (*sh)[4], int warp, int lane) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = SUM ? warp_sum(v[i]) : warp_max(v[i]);
    cons_sync();
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) sh[warp][i] = v[i];
    }
    cons_sync();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float t = SUM ? 0.f : sh[0][i];
#pragma unroll
        for (int w = SUM ? 0 : 1; w < kConsWarps; ++w) t = SUM ? t + sh[w][i] : fmaxf(t, sh[w][i]);
        v[i] = t;
    }
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
__device__ __forceinline__ void emit(const float (&xv)[W], const SProblem& P, int j, float* xs, float& sx, float& sxmy,
                                     float& xmax) {
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
        sxmy = fmaf(xv[e], my[e], sxmy);
        xmax = (xp[e] == xp[e]) ? fmaxf(xmax, fabsf(xp[e])) : __int_as_float(0x7f800000);
    }
#pragma unroll
    for (int e = 0; e < W; e += 4) *reinterpret_cast<float4*>(xs + j + e) = make_float4(xp[e], xp[e + 1], xp[e + 2], xp[e + 3]);
}

// Ask L2 for this CTA's share of the lines of a vector that the NEXT phase reads right after the grid
// barrier (model constants and last token's state: the 7 GB of weights streamed since their last use
// have pushed them out of L2).  evict_last keeps them there across tokens.
__device__ __forceinline__ void l2_fetch(const void* ptr, int bytes, int cta, int G, int tid) {
    if (ptr == nullptr) return;
    const char* p = static_cast<const char*>(ptr);
    const int lines = (bytes + 127) >> 7;
    for (int l = cta + tid * G; l < lines; l += G * kConsumers)
        asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(p + (size_t)l * 128));
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
                    const long long stage_bytes = (long long)g.kbs * g.kb_bytes;
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
    const int gid = lane >> 2, tig = lane & 3;      // fragment coordinates of the lane
    int slot = 0;
    uint32_t parity = 0;
    for (int ph = 0; ph < n_phases; ++ph) {
        const SPhase& PH = phases[ph];
        const int count = PH.count;

        // ---- prologue: every CTA builds the full quantised activation vector of each problem ----
        uint4 lnx[2];
        float mean = 0.f, rstd = 0.f;
        float xmax[4] = {0.f, 0.f, 0.f, 0.f};
        lnx[0] = lnx[1] = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int z = 0; z < kMaxPhaseProblems; ++z) {
            if (z >= count) break;
            const SProblem& P = PH.p[z];
            const int N = P.N;
            float* xs = reinterpret_cast<float*>(xq_base + P.xq_off);
            float sx = 0.f, sxmy = 0.f, xm = 0.f;
            if (P.prologue == RWKV_PRO_LN_MIX) {
                if (!P.share_ln) {
                    // LayerNorm statistics in one pass, shifted by the first element so that a large mean does
                    // not cancel (N <= 8192: two 16-byte loads per thread)
                    const float x0 = __half2float(__ldcg(static_cast<const __half*>(P.x)));
                    float st[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int j8 = (tid + i * kConsumers) * 8;
                        if (j8 < N) {
                            lnx[i] = ldcg16(P.x, j8);
                            float f[8];
                            h8_to_f(lnx[i], f);
#pragma unroll
                            for (int e = 0; e < 8; ++e) { const float d = f[e] - x0; st[0] += d; st[1] = fmaf(d, d, st[1]); }
                        }
                    }
                    cons_block_reduce4<true>(st, ctl->red, warp, lane);
                    const float md = st[0] / float(N);
                    mean = x0 + md;
                    rstd = rsqrtf(fmaxf(st[1] / float(N) - md * md, 0.f) + 1e-5f);
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
                        emit<8>(xv, P, j8, xs, sx, sxmy, xm);
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
                    emit<4>(xv, P, j, xs, sx, sxmy, xm);
                }
            } else {
                for (int j8 = tid * 8; j8 < N; j8 += kConsumers * 8) {
                    float xv[8];
                    h8_to_f(ldcg16(P.x, j8), xv);
                    emit<8>(xv, P, j8, xs, sx, sxmy, xm);
                }
            }
            sx = warp_sum(sx); sxmy = warp_sum(sxmy);
            if (lane == 0) { ctl->wsum[z][warp][0] = sx; ctl->wsum[z][warp][1] = sxmy; }
            xmax[z] = xm;
        }
        cons_block_reduce4<false>(xmax, ctl->red, warp, lane);       // also orders the x' stores before the reads below
        // quantise in place.  The 16 fp32 x' of inputs [16 g, 16 g + 16) become 64 bytes of digits in the same
        // place: plane n (the n-th signed base-256 digit) of those inputs at byte 16 n; two such groups are the
        // k-block whose A fragments the lanes with gid < 4 read as words gid * 4 + tig (+ 16).
#pragma unroll
        for (int z = 0; z < kMaxPhaseProblems; ++z) {
            if (z >= count) break;
            const SProblem& P = PH.p[z];
            const int N = P.N, npad = ((N + 31) >> 5) << 5;
            float* xs = reinterpret_cast<float*>(xq_base + P.xq_off);
            const float m = xmax[z];
            const bool finite = m < 3.0e38f;
            const float scale = (finite && m > 0.f) ? kQMax / m : 0.f;
            if (tid == 0) ctl->inv_scale[z] = !finite ? __int_as_float(0x7fc00000) : (m > 0.f ? m / kQMax : 0.f);
            long long sq = 0;
            for (int j0 = 0; j0 < npad; j0 += kConsumers * 4) {     // whole warps iterate together (npad % 32 == 0)
                const int j = j0 + tid * 4;
                uint32_t plane[4] = {0u, 0u, 0u, 0u};
                if (j < N) {                                        // N % 8 == 0: a group of four is inside or outside
                    const float4 v = *reinterpret_cast<const float4*>(xs + j);
                    const float f[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        int q = __float2int_rn(f[e] * scale);
                        sq += q;
#pragma unroll
                        for (int n = 0; n < 4; ++n) {
                            const int d = (int)(signed char)(q & 0xff);
                            plane[n] |= uint32_t(d & 0xff) << (8 * e);
                            q = (q - d) >> 8;
                        }
                    }
                }
                __syncwarp();                                       // the group's floats are read before its digits land
                if (j < npad) {
                    uint32_t* dst = reinterpret_cast<uint32_t*>(xs) + (j >> 4) * 16 + ((j & 15) >> 2);
#pragma unroll
                    for (int n = 0; n < 4; ++n) dst[n * 4] = plane[n];
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (lane == 0) ctl->wsumq[z][warp] = sq;
        }
        cons_sync();
        if (trace != nullptr && tid == 0 && cta < 2) trace[(ph * 2 + cta) * 4 + 2] = gtime();

        // what the next phase reads right after the barrier and nobody writes in this phase
        if (ph + 1 < n_phases) {
            const SPhase& NX = phases[ph + 1];
            for (int z = 0; z < NX.count; ++z) {
                const SProblem& P = NX.p[z];
                l2_fetch(P.ry, P.N * 2, cta, G, tid);
                l2_fetch(P.my, P.N * 2, cta, G, tid);
                if (P.prologue == RWKV_PRO_LN_MIX) {
                    l2_fetch(P.p0, P.N * 2, cta, G, tid); l2_fetch(P.p1, P.N * 2, cta, G, tid);
                    l2_fetch(P.p2, P.N * 2, cta, G, tid); l2_fetch(P.p3, P.N * 2, cta, G, tid);
                } else if (P.prologue == RWKV_PRO_WKV4) {
                    l2_fetch(P.f0, P.N * 4, cta, G, tid); l2_fetch(P.f1, P.N * 4, cta, G, tid);
                    l2_fetch(P.f2, P.N * 4, cta, G, tid); l2_fetch(P.f3, P.N * 4, cta, G, tid);
                    l2_fetch(P.f4, P.N * 4, cta, G, tid);
                }
            }
        }

        // ---- the matrices of the phase, one after the other ----
        for (int z = 0; z < count; ++z) {
            const SProblem& P = PH.p[z];
            const Geom g = seg_geom(P.N, P.M, cta, G);
            const uint32_t* xq = reinterpret_cast<const uint32_t*>(xq_base + P.xq_off);
            // the epilogue's operands, on their way while the matrix streams
            const int kcol = (g.u0 << 2) + tid;
            const bool fin = tid < 4 * g.Q && kcol < P.M;
            float rxk = 0.f, mxk = 0.f, auxv = 0.f, aux2v = 0.f;
            if (fin) {
                rxk = __half2float(__ldg(static_cast<const __half*>(P.rx) + kcol));
                mxk = __half2float(__ldg(static_cast<const __half*>(P.mx) + kcol));
                if (P.epilogue == RWKV_EPI_RESIDUAL || P.epilogue == RWKV_EPI_MUL_RESIDUAL)
                    auxv = __half2float(__ldcg(static_cast<const __half*>(P.aux) + kcol));
                if (P.epilogue == RWKV_EPI_MUL_RESIDUAL) aux2v = __half2float(__ldcg(static_cast<const __half*>(P.aux2) + kcol));
                if (P.epilogue == RWKV_EPI_ACC_F32) auxv = __ldcg(static_cast<const float*>(P.y) + kcol);
            }
            const int og = warp % g.wo, ks = warp / g.wo;
            const int o_first = og * g.opw;
            const int my_oct = max(0, min(g.opw, g.n_oct - o_first));
            const bool half_last = (g.Q & 1) != 0;                  // the CTA's last octet holds four columns
            int acc[kMaxOct][2];
#pragma unroll
            for (int o = 0; o < kMaxOct; ++o) acc[o][0] = acc[o][1] = 0;
            for (int s = 0; s < g.n_stages; ++s) {
                mbar_wait(s2u(&ctl->full[slot]), parity, err, gerr);
                const uint8_t* sp = ring + (size_t)slot * kSlotBytes;
                const int kb0 = s * g.kbs;
                const int nkb = min(g.kbs, g.n_kb - kb0);
                int kl = (ks - kb0 % g.wk + g.wk) % g.wk;          // first k-block of the stage that is this warp's
                for (; kl < nkb; kl += g.wk) {
                    const int kb = kb0 + kl;
                    uint32_t a0 = 0u, a2 = 0u;
                    if (gid < 4) { a0 = xq[kb * 32 + gid * 4 + tig]; a2 = xq[kb * 32 + 16 + gid * 4 + tig]; }
                    const uint2* cells = reinterpret_cast<const uint2*>(sp + (size_t)kl * g.kb_bytes) + o_first * 32 + lane;
#pragma unroll
                    for (int o = 0; o < kMaxOct; ++o) {
                        if (o < my_oct) {
                            const bool whole = !(half_last && o_first + o == g.n_oct - 1);
                            uint2 b = make_uint2(0u, 0u);
                            if (whole || lane < 16) b = cells[o * 32];
                            imma_16832(acc[o][0], acc[o][1], a0, a2, b.x, b.y);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(s2u(&ctl->empty[slot]));
                if (++slot == n_slots) { slot = 0; parity ^= 1; }
            }
            // lane (gid < 4, tig) holds digit gid of columns 2 tig, 2 tig + 1 of each of its octets: weigh the
            // digits, add them over gid (lanes 4 and 8 apart), then the K groups of warps through shared memory
            cons_sync();                    // the previous matrix's partial sums have been read
#pragma unroll
            for (int o = 0; o < kMaxOct; ++o) {
                if (o < my_oct) {
                    long long v0 = gid < 4 ? (long long)acc[o][0] << (8 * gid) : 0ll;
                    long long v1 = gid < 4 ? (long long)acc[o][1] << (8 * gid) : 0ll;
                    v0 += __shfl_xor_sync(0xffffffffu, v0, 4); v1 += __shfl_xor_sync(0xffffffffu, v1, 4);
                    v0 += __shfl_xor_sync(0xffffffffu, v0, 8); v1 += __shfl_xor_sync(0xffffffffu, v1, 8);
                    if (gid == 0) {
                        red[(warp * kMaxOct + o) * 8 + 2 * tig] = v0;
                        red[(warp * kMaxOct + o) * 8 + 2 * tig + 1] = v1;
                    }
                }
            }
            cons_sync();
            if (fin) {
                const int oc = tid >> 3, ogf = oc / g.opw, ol = oc - ogf * g.opw;
                long long tot = 0;
                for (int k2 = 0; k2 < g.wk; ++k2) tot += red[((k2 * g.wo + ogf) * kMaxOct + ol) * 8 + (tid & 7)];
                float tx = 0.f, txmy = 0.f;
                long long sq = 0;
#pragma unroll
                for (int w8 = 0; w8 < kConsWarps; ++w8) {
                    tx += ctl->wsum[z][w8][0]; txmy += ctl->wsum[z][w8][1];
                    sq += ctl->wsumq[z][w8];
                }
                // sum_j x'_j (w_jk + 1/2) = inv_scale * (sum q w + sum q / 2): one exact integer, no cancellation
                const float sdot = __ll2float_rn(2 * tot + sq) * (0.5f * ctl->inv_scale[z]);
                const float val = fmaf(rxk, sdot, fmaf(mxk, tx, txmy));
                const int k = kcol;
                __half* yh = static_cast<__half*>(P.y);
                switch (P.epilogue) {
                case RWKV_EPI_ACC_F32: static_cast<float*>(P.y)[k] = auxv + val; break;
                case RWKV_EPI_STORE: yh[k] = __float2half_rn(val); break;
                case RWKV_EPI_SIGMOID: yh[k] = __float2half_rn(1.0f / (1.0f + expf(-r16(val)))); break;
                case RWKV_EPI_RELU_SQ: { const float v = fmaxf(r16(val), 0.0f); yh[k] = __float2half_rn(v * v); break; }
                case RWKV_EPI_RESIDUAL: yh[k] = __float2half_rn(r16(auxv + r16(val)) * P.out_scale); break;
                case RWKV_EPI_MUL_RESIDUAL: yh[k] = __float2half_rn(r16(auxv + r16(aux2v * r16(val))) * P.out_scale); break;
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

// One thread per 8-byte cell: k-block kb, octet o, lane -> the B fragment of that lane, i.e. column
// 8 o + lane / 4 of the CTA, input rows 32 kb + 4 (lane % 4) + {0..3} and the same 16 rows further.
__global__ void mm8_stream_pack_kernel(PackArgs a, uint8_t* wstream) {
    const int cta = blockIdx.y;
    const Geom g = seg_geom(a.N, a.M, cta, a.G);
    if (g.Q == 0) return;
    uint2* dst = reinterpret_cast<uint2*>(wstream + a.off[cta]);
    const int per_kb = 16 * g.Q;
    const long long cells = (long long)g.n_kb * per_kb;
    for (long long cell = blockIdx.x * (long long)blockDim.x + threadIdx.x; cell < cells; cell += (long long)gridDim.x * blockDim.x) {
        const int kb = int(cell / per_kb), rem = int(cell - (long long)kb * per_kb);
        const int o = rem >> 5, lane = rem & 31;
        const int col = (g.u0 << 2) + 8 * o + (lane >> 2);
        const int r0 = 32 * kb + 4 * (lane & 3);
        uint32_t b[2] = {0u, 0u};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = r0 + 16 * h + i;
                if (row < a.N && col < a.M) b[h] |= uint32_t(a.w[(long long)row * a.w_stride + col]) << (8 * i);
            }
        }
        dst[cell] = make_uint2(b[0], b[1]);
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
    if (((q.M + 3) / 4 + G - 1) / G > kSlotBytes / 128) return false;
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
        long long max_cells = 0;
        for (int c = 0; c < n_ctas; ++c) {
            const Geom g = seg_geom(q.N, q.M, c, n_ctas);
            a.off[c] = base[c] + run[c];
            run[c] += g.bytes;
            if (g.bytes / 8 > max_cells) max_cells = g.bytes / 8;
        }
        if (max_cells == 0) continue;
        const int bx = (max_cells + 255) / 256 > 64 ? 64 : int((max_cells + 255) / 256);
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
            off += ((q.N + 31) >> 5) * 128;        // 4 bytes per input, whole k-blocks of 32
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
