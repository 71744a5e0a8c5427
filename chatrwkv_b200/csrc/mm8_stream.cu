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
// signed base-256 digits, stored as digit planes.  dp4a multiplies the four digits-n of four
// consecutive inputs with the four raw codes of one column: exact 32-bit sums per digit (|d w| <=
// 32640 per product, so 65536 inputs cannot overflow), weighted by 256^n in 64-bit integers at the
// end.  The streamed part of mm8_one (operators.cu:224-230) is therefore computed exactly for the
// quantised x', whose relative error (2^-24 of fp32 for large entries, 2^-30 of the largest entry
// for small ones) is that of an fp32 product; no result depends on a summation order.
// (Measured and dropped: the same products on mma.sync.m16n8k32.s8.u8 -- digit planes as the rows of
// A, eight columns of codes as B -- ran at ~22 clocks per instruction and SM on the B200, half the
// speed of the dp2a/dp4a forms.)
#include "common.cuh"

namespace {

constexpr int kConsumers = 512;
constexpr int kConsWarps = kConsumers / 32;
constexpr int kStreamThreads = kConsumers + 32;          // + the producer warp
constexpr int kIter = 2;                                 // 16-byte cells per thread and stage
constexpr int kSlotBytes = kIter * kConsumers * 16;      // 16 KB
constexpr int kRedBytes = 128 * 4 * 8;                   // [<= 128 subgroups][4 columns] 64-bit sums
constexpr int kMaxSlots = 12;
constexpr int kMaxCtas = 160;
constexpr int kMaxPhaseProblems = 4;
constexpr int kMaxSegments = 448;                        // matrices per step (the producer's list lives in shared memory)
// Largest |q| by number of digit planes multiplied: the digits above the last plane are then zero.
__host__ __device__ constexpr float qmax_for(int planes) { return planes >= 4 ? 1.0e9f : planes == 3 ? 8.0e6f : 32000.0f; }
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
    // the layout of the matrix for a CTA (seg_geom), tabulated by the host: CTAs below `rem` own base + 1 quads
    int base, rem;
    int gSG[2], gGPI[2], gTA[2], gcells[2], gstages[2];
};

struct SPhase {
    int count;
    int ln_shared;      // every problem is RWKV_PRO_LN_MIX on the same x and LayerNorm (up to 8192 inputs)
    SProblem p[kMaxPhaseProblems];
    int pad[2];
};
static_assert(sizeof(SPhase) % 16 == 0, "phase records are copied in 16-byte pieces");

struct STable {      // 16-byte multiple: the phase records that follow are copied in 16-byte pieces
    int n_phases, n_ctas, xq_bytes, n_slots;
    int planes, n_segments, pad1, pad2; // digit planes the matrices are multiplied with (2, 3 or 4); matrices per step
    long long cta_base[kMaxCtas];       // byte offset of every CTA's region in the weight stream
    // SPhase phases[n_phases] follow
};

static_assert(sizeof(STable) % 16 == 0, "phase records start 16-byte aligned");

// How one matrix is laid out for one CTA.  A cell is 16 bytes: 4 consecutive inputs ("k-group") x 4
// consecutive columns ("quad"), one 32-bit word per column holding the 4 inputs' codes.  The CTA
// owns Q quads.  A subgroup of SG lanes works on one quad; there are as many subgroups per quad as
// fit 512 threads, so an iteration of the CTA covers GPI = SG * subgroups k-groups of every quad, and
// thread t's cell of iteration `it` sits at byte (it * TA + t) * 16 of the matrix's segment.
struct Geom {
    int Q;              // column quads owned by this CTA
    int u0;             // first quad
    int SG;             // lanes that share a quad inside a warp (4, 8, 16 or 32)
    int GPI;            // k-groups per iteration
    int TA;             // active threads = Q * GPI
    int kg;             // k-groups, rounded up to a multiple of SG
    int cells;          // kg * Q
    int n_stages;
    long long bytes;    // cells * 16
};

__host__ __device__ inline Geom seg_geom(int N, int M, int cta, int G) {
    Geom g;
    const int U = (M + 3) >> 2;
    const int base = U / G, rem = U % G;
    g.Q = base + (cta < rem ? 1 : 0);
    g.u0 = cta * base + (cta < rem ? cta : rem);
    g.SG = 4; g.GPI = 0; g.TA = 0; g.kg = 0; g.cells = 0; g.n_stages = 0; g.bytes = 0;
    if (g.Q == 0 || g.Q > kConsumers / 4) return g;       // more than 128 quads per CTA: not planned (see plan)
    int best_ta = 0;
    for (int sg = 32; sg >= 4; sg >>= 1) {
        const int nsub = (kConsumers / sg) / g.Q;
        const int ta = nsub * g.Q * sg;
        if (ta > best_ta) { best_ta = ta; g.SG = sg; }
    }
    g.TA = best_ta;
    g.GPI = best_ta / g.Q;
    const int kg = (N + 3) >> 2;
    g.kg = (kg + g.SG - 1) / g.SG * g.SG;
    g.cells = g.kg * g.Q;
    const int per_stage = kIter * g.TA;
    g.n_stages = (g.cells + per_stage - 1) / per_stage;
    g.bytes = (long long)g.cells * 16;
    return g;
}

// seg_geom from the table the host put into the problem record (no divisions on the device)
__device__ __forceinline__ Geom seg_geom_dev(const SProblem& P, int cta) {
    Geom g;
    const int v = cta < P.rem ? 1 : 0;
    g.Q = P.base + v;
    g.u0 = cta * P.base + (v ? cta : P.rem);
    g.SG = P.gSG[v]; g.GPI = P.gGPI[v]; g.TA = P.gTA[v]; g.cells = P.gcells[v]; g.n_stages = P.gstages[v];
    g.kg = 0;
    g.bytes = (long long)g.cells * 16;
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

__device__ __forceinline__ unsigned short ld_cg_u16(const void* p) {
    unsigned short v;
    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_cg_f32(const void* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
// c + sum_i a.byte_i (signed digit) * b.byte_i (unsigned code)
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// The cells of one stage: acc[column][digit] += digits of 4 inputs . codes of 4 inputs, for P digit planes.
template <int P>
__device__ __forceinline__ void stage_math(int (&acc)[4][4], const uint4 (&w)[kIter], const uint4 (&xv)[kIter]) {
#pragma unroll
    for (int r = 0; r < kIter; ++r) {
        const uint32_t wc[4] = {w[r].x, w[r].y, w[r].z, w[r].w};
        const uint32_t dn[4] = {xv[r].x, xv[r].y, xv[r].z, xv[r].w};
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int n = 0; n < P; ++n) acc[c][n] = dp4a_su(dn[n], wc[c], acc[c][n]);
    }
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
    float tot_x[kMaxPhaseProblems], tot_xmy[kMaxPhaseProblems];     // sums over all inputs, made once per problem
    long long tot_q[kMaxPhaseProblems];
    float red[2][kConsWarps][4];
    int err;
    int pad[3];
    alignas(16) SPhase phase[2];        // the current and the next phase's records, copied from the table ahead of use
    uint2 sched[kMaxSegments];          // the producer's list: {cells, TA | stages << 16} of every matrix for this CTA
};

// Reductions over the 512 consumer threads.  Two scratch buffers alternate (`flip`), so one barrier per
// reduction is enough: a buffer is rewritten only after every thread has passed the barrier of the
// reduction in between, i.e. after it has finished reading.
__device__ __forceinline__ void cons_block_sum2(float& a, float& b, float (*sh)[kConsWarps][4], int& flip, int warp, int lane) {
    a = warp_sum(a); b = warp_sum(b);
    float (*buf)[4] = sh[flip];
    flip ^= 1;
    if (lane == 0) { buf[warp][0] = a; buf[warp][1] = b; }
    cons_sync();
    a = 0.f; b = 0.f;
#pragma unroll
    for (int w = 0; w < kConsWarps; ++w) { a += buf[w][0]; b += buf[w][1]; }
}
// maxima of four non-negative values (their bit patterns order like the values; +inf stays the largest)
__device__ __forceinline__ void cons_block_max4(float (&v)[4], float (*sh)[kConsWarps][4], int& flip, int warp, int lane) {
    float (*buf)[4] = sh[flip];
    flip ^= 1;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const unsigned m = __reduce_max_sync(0xffffffffu, __float_as_uint(v[i]));
        if (lane == 0) buf[warp][i] = __uint_as_float(m);
    }
    cons_sync();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float t = buf[0][i];
#pragma unroll
        for (int w = 1; w < kConsWarps; ++w) t = fmaxf(t, buf[w][i]);
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
__device__ __forceinline__ void emit_with(const float (&xv)[W], const float (&ry)[W], const float (&my)[W], int j, float* xs,
                                          float& sx, float& sxmy, float& xmax) {
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
// The same for 8 activations held as four half2 (xv); ry, my as loaded.  A non-finite activation is caught
// by the caller through the sum.
__device__ __forceinline__ void emit_h8(const uint4& xv, const uint4& ryv, const uint4& myv, int j, float* xs,
                                        float& sx, float& sxmy, float& xmax) {
    const __half2* hx = reinterpret_cast<const __half2*>(&xv);
    const __half2* hr = reinterpret_cast<const __half2*>(&ryv);
    const __half2* hm = reinterpret_cast<const __half2*>(&myv);
    float xp[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 x = __half22float2(hx[e]), r = __half22float2(hr[e]), m = __half22float2(hm[e]);
        xp[2 * e] = x.x * r.x; xp[2 * e + 1] = x.y * r.y;
        sx += x.x + x.y;
        sxmy = fmaf(x.x, m.x, sxmy); sxmy = fmaf(x.y, m.y, sxmy);
        xmax = fmaxf(xmax, fmaxf(fabsf(xp[2 * e]), fabsf(xp[2 * e + 1])));
    }
    *reinterpret_cast<float4*>(xs + j) = make_float4(xp[0], xp[1], xp[2], xp[3]);
    *reinterpret_cast<float4*>(xs + j + 4) = make_float4(xp[4], xp[5], xp[6], xp[7]);
}
// token-shift mix of 8 LayerNorm outputs xx with the previous token's sv in fp16 arithmetic, one rounding per
// operation as the reference's tensor ops have: mode 0 xx*mix + sv*(1-mix) (pkg/model.py:986, 1036-1038),
// mode 1 xx + (sv-xx)*mix (pkg/model.py:1009-1011)
__device__ __forceinline__ uint4 mix_h8(const uint4& xx, const uint4& sv, const uint4& mv, int mode) {
    uint4 out;
    const __half2* a = reinterpret_cast<const __half2*>(&xx);
    const __half2* b = reinterpret_cast<const __half2*>(&sv);
    const __half2* m = reinterpret_cast<const __half2*>(&mv);
    __half2* o = reinterpret_cast<__half2*>(&out);
    const __half2 one = __floats2half2_rn(1.0f, 1.0f);
#pragma unroll
    for (int e = 0; e < 4; ++e)
        o[e] = mode == 0 ? __hadd2(__hmul2(a[e], m[e]), __hmul2(b[e], __hsub2(one, m[e])))
                         : __hadd2(a[e], __hmul2(__hsub2(b[e], a[e]), m[e]));
    return out;
}
// LayerNorm of 8 inputs: fp32 arithmetic, one rounding to fp16 at the end
__device__ __forceinline__ uint4 ln_h8(const uint4& x, const uint4& lw, const uint4& lb, float mean, float rstd) {
    float f[8], w[8], b[8], o[8];
    h8_to_f(x, f); h8_to_f(lw, w); h8_to_f(lb, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = (f[e] - mean) * rstd * w[e] + b[e];
    return f_to_h8(o);
}
__device__ __forceinline__ void h4_to_f(const uint2& v, float (&f)[4]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int e = 0; e < 2; ++e) { const float2 t = __half22float2(h[e]); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
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
    // The table lives in global memory that the weight stream pushes out of L2 between uses: the producer's
    // list of matrices and the first phase record go to shared memory now, later phase records one phase ahead.
    const int n_segments = table->n_segments;
    {
        int k = 0;
        for (int ph = 0; ph < n_phases; ++ph) {
            const int count = phases[ph].count;
            for (int z = 0; z < count; ++z, ++k) {
                if ((k % kStreamThreads) == tid) {
                    const Geom g = seg_geom_dev(phases[ph].p[z], cta);
                    ctl->sched[k] = make_uint2((unsigned)g.cells, (unsigned)g.TA | ((unsigned)g.n_stages << 16));
                }
            }
        }
    }
    for (int i = tid; i < int(sizeof(SPhase) / 16); i += kStreamThreads)
        reinterpret_cast<uint4*>(&ctl->phase[0])[i] = __ldg(reinterpret_cast<const uint4*>(&phases[0]) + i);
    __syncthreads();
    volatile int* err = &ctl->err;

    if (warp == kConsWarps) {
        // ================= producer: one thread walks this CTA's region of the stream =================
        if (lane == 0) {
            const uint8_t* src = wstream + table->cta_base[cta];
            int slot = 0;
            uint32_t parity = 1;            // a fresh mbarrier passes a wait on parity 1: every slot starts empty
            for (int k = 0; k < n_segments; ++k) {
                const uint2 sc = ctl->sched[k];
                const long long seg_bytes = (long long)sc.x * 16;
                const long long stage_bytes = (long long)kIter * (sc.y & 0xffffu) * 16;
                const int n_stages = int(sc.y >> 16);
                for (int s = 0; s < n_stages; ++s) {
                    const long long left = seg_bytes - s * stage_bytes;
                    const uint32_t bytes = (uint32_t)(left < stage_bytes ? left : stage_bytes);
                    mbar_wait(s2u(&ctl->empty[slot]), parity, err, gerr);
                    mbar_expect_tx(s2u(&ctl->full[slot]), bytes);
                    bulk_g2s(s2u(ring + (size_t)slot * kSlotBytes), src + s * stage_bytes, bytes, s2u(&ctl->full[slot]));
                    if (++slot == n_slots) { slot = 0; parity ^= 1; }
                }
                src += seg_bytes;
            }
        }
        return;
    }

    // ================= consumers =================
    const int planes = table->planes;
    int flip = 0;
    int slot = 0;
    uint32_t parity = 0;
    for (int ph = 0; ph < n_phases; ++ph) {
        const SPhase& PH = ctl->phase[ph & 1];
        const int count = PH.count;

        // ---- prologue: every CTA builds the full quantised activation vector of each problem ----
        // All global loads of a pass are issued before the first use, so that a pass costs one trip to L2.
        float xmax[4] = {0.f, 0.f, 0.f, 0.f};
        if (PH.ln_shared) {
            // LayerNorm + token-shift mixes of one residual vector for up to four matrices (r/k/v(/g), ffn r/k,
            // head).  Thread t holds inputs [8 t, 8 t + 8) and, above 4096 inputs, [8 t + 4096, ...).
            const SProblem& P0 = PH.p[0];
            const int N = P0.N;
            const bool mixes = P0.mode != 2;
            uint4 lnx[2];
            lnx[0] = lnx[1] = make_uint4(0, 0, 0, 0);
            float sxz[4] = {0.f, 0.f, 0.f, 0.f}, smz[4] = {0.f, 0.f, 0.f, 0.f};
            const float x0 = __half2float(__ldcg(static_cast<const __half*>(P0.x)));
            // statistics in one pass, shifted by the first element so that a large mean does not cancel
            float s1 = 0.f, s2 = 0.f;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int j8 = (tid + i * kConsumers) * 8;
                if (j8 < N) {
                    lnx[i] = ldcg16(P0.x, j8);
                    float f[8];
                    h8_to_f(lnx[i], f);
#pragma unroll
                    for (int e = 0; e < 8; ++e) { const float d = f[e] - x0; s1 += d; s2 = fmaf(d, d, s2); }
                }
            }
            cons_block_sum2(s1, s2, ctl->red, flip, warp, lane);
            if (trace != nullptr && tid == 0 && cta < 2) trace[(ph * 2 + cta) * 16 + 4] = gtime();
            const float md = s1 / float(N);
            const float mean = x0 + md;
            const float rstd = rsqrtf(fmaxf(s2 / float(N) - md * md, 0.f) + 1e-5f);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int j8 = (tid + i * kConsumers) * 8;
                if (j8 < N) {
                    const uint4 xx = ln_h8(lnx[i], ldg16(P0.p0, j8), ldg16(P0.p1, j8), mean, rstd);
                    if (P0.q0 != nullptr && ((j8 >> 3) % G) == cta) *reinterpret_cast<uint4*>(static_cast<__half*>(P0.q0) + j8) = xx;
                    uint4 sv = make_uint4(0, 0, 0, 0);
                    if (mixes) sv = ldcg16(P0.p2, j8);
#pragma unroll
                    for (int z = 0; z < kMaxPhaseProblems; ++z) {
                        if (z < count) {
                            const SProblem& P = PH.p[z];
                            const uint4 xv = mixes ? mix_h8(xx, sv, ldg16(P.p3, j8), P0.mode) : xx;
                            emit_h8(xv, ldg16(P.ry, j8), ldg16(P.my, j8), j8, reinterpret_cast<float*>(xq_base + P.xq_off),
                                    sxz[z], smz[z], xmax[z]);
                        }
                    }
                }
            }
#pragma unroll
            for (int z = 0; z < kMaxPhaseProblems; ++z) {
                if (z < count) {
                    if (!(fabsf(sxz[z]) <= 3.0e38f)) xmax[z] = __int_as_float(0x7f800000);   // an inf or NaN activation
                    const float a1 = warp_sum(sxz[z]), a2 = warp_sum(smz[z]);
                    if (lane == 0) { ctl->wsum[z][warp][0] = a1; ctl->wsum[z][warp][1] = a2; }
                }
            }
        } else {
#pragma unroll
            for (int z = 0; z < kMaxPhaseProblems; ++z) {
                if (z >= count) break;
                const SProblem& P = PH.p[z];
                const int N = P.N;
                float* xs = reinterpret_cast<float*>(xq_base + P.xq_off);
                float sx = 0.f, sxmy = 0.f, xm = 0.f;
                if (P.prologue == RWKV_PRO_WKV4) {           // pkg/model.py:1041-1055, four channels per thread and pass
#pragma unroll 1
                    for (int j = tid * 4; j < N; j += kConsumers * 4) {
                        const uint2 r2 = __ldcg(reinterpret_cast<const uint2*>(static_cast<const __half*>(P.x) + j));
                        const uint2 k2 = __ldcg(reinterpret_cast<const uint2*>(static_cast<const __half*>(P.p0) + j));
                        const uint2 v2 = __ldcg(reinterpret_cast<const uint2*>(static_cast<const __half*>(P.p1) + j));
                        const float4 a4 = __ldcg(reinterpret_cast<const float4*>(P.f2 + j));
                        const float4 b4 = __ldcg(reinterpret_cast<const float4*>(P.f3 + j));
                        const float4 p4 = __ldcg(reinterpret_cast<const float4*>(P.f4 + j));
                        const float4 d4 = __ldg(reinterpret_cast<const float4*>(P.f0 + j));
                        const float4 f4 = __ldg(reinterpret_cast<const float4*>(P.f1 + j));
                        const uint2 ry2 = __ldg(reinterpret_cast<const uint2*>(static_cast<const __half*>(P.ry) + j));
                        const uint2 my2 = __ldg(reinterpret_cast<const uint2*>(static_cast<const __half*>(P.my) + j));
                        const float aa[4] = {a4.x, a4.y, a4.z, a4.w}, bb[4] = {b4.x, b4.y, b4.z, b4.w}, pp[4] = {p4.x, p4.y, p4.z, p4.w};
                        const float td[4] = {d4.x, d4.y, d4.z, d4.w}, tf[4] = {f4.x, f4.y, f4.z, f4.w};
                        float rr[4], kk[4], vv[4], ry[4], my[4], xv[4], na[4], nb[4], np[4];
                        h4_to_f(r2, rr); h4_to_f(k2, kk); h4_to_f(v2, vv); h4_to_f(ry2, ry); h4_to_f(my2, my);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float ww = tf[e] + kk[e];
                            float p = fmaxf(pp[e], ww);
                            float e1 = expf(pp[e] - p), e2 = expf(ww - p);
                            const float wkv = r16((e1 * aa[e] + e2 * vv[e]) / (e1 * bb[e] + e2));
                            ww = td[e] + pp[e];
                            p = fmaxf(ww, kk[e]);
                            e1 = expf(ww - p); e2 = expf(kk[e] - p);
                            na[e] = e1 * aa[e] + e2 * vv[e];
                            nb[e] = e1 * bb[e] + e2;
                            np[e] = p;
                            xv[e] = r16(rr[e] * wkv);
                        }
                        if (((j >> 3) % G) == cta) {
                            *reinterpret_cast<float4*>(P.g0 + j) = make_float4(na[0], na[1], na[2], na[3]);
                            *reinterpret_cast<float4*>(P.g1 + j) = make_float4(nb[0], nb[1], nb[2], nb[3]);
                            *reinterpret_cast<float4*>(P.g2 + j) = make_float4(np[0], np[1], np[2], np[3]);
                        }
                        emit_with<4>(xv, ry, my, j, xs, sx, sxmy, xm);
                    }
                } else if (P.prologue == RWKV_PRO_LN_MIX) {   // a LayerNorm problem outside a shared phase: two passes over x
                    float s1 = 0.f, s2 = 0.f;
                    const float x0 = __half2float(__ldcg(static_cast<const __half*>(P.x)));
                    for (int j8 = tid * 8; j8 < N; j8 += kConsumers * 8) {
                        float f[8];
                        h8_to_f(ldcg16(P.x, j8), f);
#pragma unroll
                        for (int e = 0; e < 8; ++e) { const float d = f[e] - x0; s1 += d; s2 = fmaf(d, d, s2); }
                    }
                    cons_block_sum2(s1, s2, ctl->red, flip, warp, lane);
                    const float md = s1 / float(N), mean = x0 + md;
                    const float rstd = rsqrtf(fmaxf(s2 / float(N) - md * md, 0.f) + 1e-5f);
                    for (int j8 = tid * 8; j8 < N; j8 += kConsumers * 8) {
                        uint4 xv = ln_h8(ldcg16(P.x, j8), ldg16(P.p0, j8), ldg16(P.p1, j8), mean, rstd);
                        if (P.q0 != nullptr && ((j8 >> 3) % G) == cta) *reinterpret_cast<uint4*>(static_cast<__half*>(P.q0) + j8) = xv;
                        if (P.mode != 2) xv = mix_h8(xv, ldcg16(P.p2, j8), ldg16(P.p3, j8), P.mode);
                        emit_h8(xv, ldg16(P.ry, j8), ldg16(P.my, j8), j8, xs, sx, sxmy, xm);
                    }
                    if (!(fabsf(sx) <= 3.0e38f)) xm = __int_as_float(0x7f800000);
                } else {
#pragma unroll 4
                    for (int j8 = tid * 8; j8 < N; j8 += kConsumers * 8)
                        emit_h8(ldcg16(P.x, j8), ldg16(P.ry, j8), ldg16(P.my, j8), j8, xs, sx, sxmy, xm);
                    if (!(fabsf(sx) <= 3.0e38f)) xm = __int_as_float(0x7f800000);
                }
                sx = warp_sum(sx); sxmy = warp_sum(sxmy);
                if (lane == 0) { ctl->wsum[z][warp][0] = sx; ctl->wsum[z][warp][1] = sxmy; }
                xmax[z] = xm;
            }
        }
        if (trace != nullptr && tid == 0 && cta < 2) trace[(ph * 2 + cta) * 16 + 5] = gtime();
        cons_block_max4(xmax, ctl->red, flip, warp, lane);           // its barrier also orders the x' stores before the reads below
        if (trace != nullptr && tid == 0 && cta < 2) trace[(ph * 2 + cta) * 16 + 6] = gtime();
        // quantise in place: the 4 fp32 x' of a k-group become its 4 digit planes (word n = the n-th signed
        // base-256 digit of the 4 inputs), which is what one dp4a multiplies with a column's 4 codes.
        // q + 0x80808080 has the digits + 128 as its plain bytes; a 4 x 4 byte transpose makes the planes.
        const float qmax = qmax_for(planes);
#pragma unroll
        for (int z = 0; z < kMaxPhaseProblems; ++z) {
            if (z >= count) break;
            const SProblem& P = PH.p[z];
            const int N = P.N, npad = (((N + 3) >> 2) + 31 & ~31) << 2;
            float* xs = reinterpret_cast<float*>(xq_base + P.xq_off);
            const float m = xmax[z];
            const bool finite = m < 3.0e38f;
            const float scale = (finite && m > 0.f) ? qmax / m : 0.f;
            if (tid == 0) ctl->inv_scale[z] = !finite ? __int_as_float(0x7fc00000) : (m > 0.f ? m / qmax : 0.f);
            long long sq = 0;
#pragma unroll 2
            for (int j = tid * 4; j < npad; j += kConsumers * 4) {
                uint4 planes4 = make_uint4(0u, 0u, 0u, 0u);
                if (j < N) {                                        // N % 8 == 0: a group of four is inside or outside
                    const float4 v = *reinterpret_cast<const float4*>(xs + j);
                    const int q0 = __float2int_rn(v.x * scale), q1 = __float2int_rn(v.y * scale);
                    const int q2 = __float2int_rn(v.z * scale), q3 = __float2int_rn(v.w * scale);
                    sq += (long long)q0 + q1 + q2 + q3;
                    const uint32_t u0 = (uint32_t(q0) + 0x80808080u) ^ 0x80808080u, u1 = (uint32_t(q1) + 0x80808080u) ^ 0x80808080u;
                    const uint32_t u2 = (uint32_t(q2) + 0x80808080u) ^ 0x80808080u, u3 = (uint32_t(q3) + 0x80808080u) ^ 0x80808080u;
                    const uint32_t t0 = __byte_perm(u0, u1, 0x5140), t1 = __byte_perm(u2, u3, 0x5140);
                    const uint32_t t2 = __byte_perm(u0, u1, 0x7362), t3 = __byte_perm(u2, u3, 0x7362);
                    planes4 = make_uint4(__byte_perm(t0, t1, 0x5410), __byte_perm(t0, t1, 0x7632),
                                         __byte_perm(t2, t3, 0x5410), __byte_perm(t2, t3, 0x7632));
                }
                *reinterpret_cast<uint4*>(xs + j) = planes4;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (lane == 0) ctl->wsumq[z][warp] = sq;
        }
        cons_sync();
        if (warp < count) {             // warp z adds the 16 per-warp sums of problem z (fixed tree: same bits in every CTA)
            float a1 = lane < kConsWarps ? ctl->wsum[warp][lane][0] : 0.f, a2 = lane < kConsWarps ? ctl->wsum[warp][lane][1] : 0.f;
            long long aq = lane < kConsWarps ? ctl->wsumq[warp][lane] : 0ll;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) {
                a1 += __shfl_xor_sync(0xffffffffu, a1, o); a2 += __shfl_xor_sync(0xffffffffu, a2, o);
                aq += __shfl_xor_sync(0xffffffffu, aq, o);
            }
            if (lane == 0) { ctl->tot_x[warp] = a1; ctl->tot_xmy[warp] = a2; ctl->tot_q[warp] = aq; }
        }
        if (trace != nullptr && tid == 0 && cta < 2) trace[(ph * 2 + cta) * 16 + 2] = gtime();

        // what the next phase reads right after the barrier and nobody writes in this phase
        if (ph + 1 < n_phases) {
            // the next phase's record, for after the barrier (its buffer was last read in phase ph - 1)
            for (int i = tid; i < int(sizeof(SPhase) / 16); i += kConsumers)
                reinterpret_cast<uint4*>(&ctl->phase[(ph + 1) & 1])[i] = __ldg(reinterpret_cast<const uint4*>(&phases[ph + 1]) + i);
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
            const Geom g = seg_geom_dev(P, cta);
            const bool tr = trace != nullptr && tid == 0 && cta < 2 && z == 0;
            if (tr) trace[(ph * 2 + cta) * 16 + 8] = gtime();
            // the epilogue's operands, on their way while the matrix streams
            const int kcol = (g.u0 << 2) + tid;
            const bool fin = tid < 4 * g.Q && kcol < P.M;
            float rxk = 0.f, mxk = 0.f, auxv = 0.f, aux2v = 0.f;
            // (volatile loads: issued here, not where the values are used after the last stage)
            unsigned short h_rx = 0, h_mx = 0, h_aux = 0, h_aux2 = 0;
            if (fin) {
                h_rx = ld_cg_u16(static_cast<const __half*>(P.rx) + kcol);
                h_mx = ld_cg_u16(static_cast<const __half*>(P.mx) + kcol);
                if (P.epilogue == RWKV_EPI_RESIDUAL || P.epilogue == RWKV_EPI_MUL_RESIDUAL) h_aux = ld_cg_u16(static_cast<const __half*>(P.aux) + kcol);
                if (P.epilogue == RWKV_EPI_MUL_RESIDUAL) h_aux2 = ld_cg_u16(static_cast<const __half*>(P.aux2) + kcol);
                if (P.epilogue == RWKV_EPI_ACC_F32) auxv = ld_cg_f32(static_cast<const float*>(P.y) + kcol);
            }
            const uint4* xq = reinterpret_cast<const uint4*>(xq_base + P.xq_off);
            const int sub = tid / g.SG, lane_in = tid % g.SG;
            const bool active = tid < g.TA;
            const int gg = active ? (sub / g.Q) * g.SG + lane_in : 0;      // this thread's k-group within an iteration
            int acc[4][4];                                                  // [column][digit]
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int n = 0; n < 4; ++n) acc[c][n] = 0;
            const int n_full = g.TA > 0 ? g.cells / (kIter * g.TA) : 0;    // stages in which every active thread has kIter cells
            const uint4* xp = xq + gg;
            for (int s = 0; s < g.n_stages; ++s) {
                mbar_wait(s2u(&ctl->full[slot]), parity, err, gerr);
                if (tr && s == 0) trace[(ph * 2 + cta) * 16 + 9] = gtime();
                const uint4* sp = reinterpret_cast<const uint4*>(ring + (size_t)slot * kSlotBytes) + tid;
                uint4 w[kIter], xv[kIter];
                if (s < n_full) {
                    if (active) {
#pragma unroll
                        for (int r = 0; r < kIter; ++r) { w[r] = sp[r * g.TA]; xv[r] = xp[r * g.GPI]; }
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < kIter; ++r) {
                        const bool ok = active && (s * kIter + r) * g.TA + tid < g.cells;
                        w[r] = ok ? sp[r * g.TA] : make_uint4(0, 0, 0, 0);
                        xv[r] = ok ? xp[r * g.GPI] : make_uint4(0, 0, 0, 0);
                    }
                }
                xp += kIter * g.GPI;
                if (active) {
                    if (planes >= 4) stage_math<4>(acc, w, xv);
                    else if (planes == 3) stage_math<3>(acc, w, xv);
                    else stage_math<2>(acc, w, xv);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(s2u(&ctl->empty[slot]));
                if (++slot == n_slots) { slot = 0; parity ^= 1; }
            }
            // this thread's exact sums for its four columns; add the lanes of the subgroup, then the
            // subgroups of a quad through shared memory
            long long S[4];
#pragma unroll
            for (int c = 0; c < 4; ++c)
                S[c] = (long long)acc[c][0] + ((long long)acc[c][1] << 8) + ((long long)acc[c][2] << 16) + ((long long)acc[c][3] << 24);
            for (int o = g.SG >> 1; o > 0; o >>= 1) {
#pragma unroll
                for (int c = 0; c < 4; ++c) S[c] += __shfl_xor_sync(0xffffffffu, S[c], o);
            }
            if (tr) trace[(ph * 2 + cta) * 16 + 10] = gtime();
            cons_sync();                    // the previous matrix's partial sums have been read
            if (tr) trace[(ph * 2 + cta) * 16 + 11] = gtime();
            if (active && lane_in == 0) {
#pragma unroll
                for (int c = 0; c < 4; ++c) red[sub * 4 + c] = S[c];
            }
            cons_sync();
            if (tr) trace[(ph * 2 + cta) * 16 + 12] = gtime();
            if (fin) {
                rxk = __half2float(__ushort_as_half(h_rx));
                mxk = __half2float(__ushort_as_half(h_mx));
                if (P.epilogue == RWKV_EPI_RESIDUAL || P.epilogue == RWKV_EPI_MUL_RESIDUAL) auxv = __half2float(__ushort_as_half(h_aux));
                aux2v = __half2float(__ushort_as_half(h_aux2));
                const int qq = tid >> 2, i = tid & 3;
                const int nrep = g.GPI / g.SG;
                long long tot = 0;
                for (int rep = 0; rep < nrep; ++rep) tot += red[(rep * g.Q + qq) * 4 + i];
                const float tx = ctl->tot_x[z], txmy = ctl->tot_xmy[z];
                const long long sq = ctl->tot_q[z];
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
        if (trace != nullptr && tid == 0 && cta < 2) trace[(ph * 2 + cta) * 16 + 3] = gtime();

        // ---- grid barrier: the phase's results are complete and visible before anyone reads them ----
        if (ph + 1 < n_phases) {
            cons_sync();
            if (tid == 0) {
                asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(gbar) : "memory");
                if (trace != nullptr && cta < 2) trace[(ph * 2 + cta) * 16 + 0] = gtime();
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
                if (trace != nullptr && cta < 2) trace[(ph * 2 + cta) * 16 + 1] = gtime();
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

// One thread per 16-byte cell.
__global__ void mm8_stream_pack_kernel(PackArgs a, uint8_t* wstream) {
    const int cta = blockIdx.y;
    const Geom g = seg_geom(a.N, a.M, cta, a.G);
    if (g.Q == 0) return;
    uint4* dst = reinterpret_cast<uint4*>(wstream + a.off[cta]);
    for (int cell = blockIdx.x * blockDim.x + threadIdx.x; cell < g.cells; cell += gridDim.x * blockDim.x) {
        const int it = cell / g.TA, t = cell - it * g.TA;
        const int sub = t / g.SG, lane_in = t % g.SG;
        const int q = sub % g.Q, gg = (sub / g.Q) * g.SG + lane_in;
        const int r0 = 4 * (it * g.GPI + gg), c0 = (g.u0 + q) * 4;
        uint32_t wc[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = r0 + i, col = c0 + c;
                if (row < a.N && col < a.M) wc[c] |= uint32_t(a.w[(long long)row * a.w_stride + col]) << (8 * i);
            }
        }
        dst[cell] = make_uint4(wc[0], wc[1], wc[2], wc[3]);
    }
}

int g_stream_planes = 4;     // digit planes tables are planned with (process-wide tuning hook)

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
    return true;
}

}  // namespace

extern "C" int rwkv_mm8_stream_ctas(void) { return stream_ctas(); }

extern "C" void rwkv_mm8_stream_set_planes(int planes) { g_stream_planes = planes < 2 ? 2 : planes > 4 ? 4 : planes; }

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
            if (g.cells > max_cells) max_cells = g.cells;
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
    T->planes = g_stream_planes;
    {
        int total = 0;
        for (int ph = 0; ph < n_phases; ++ph) total += counts[ph];
        if (total > kMaxSegments) return RWKV_ERR_UNSUPPORTED;
        T->n_segments = total;
    }
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
            {
                const int U = (q.M + 3) >> 2;
                P.base = U / n_ctas; P.rem = U % n_ctas;
                for (int v = 0; v < 2; ++v) {
                    // a CTA index that owns base + v quads (any one: the layout depends on the quad count only)
                    const int c = v ? 0 : n_ctas - 1;
                    const Geom gg = seg_geom(q.N, q.M, c, n_ctas);
                    const bool ok = gg.Q == P.base + v;
                    P.gSG[v] = ok ? gg.SG : 4; P.gGPI[v] = ok ? gg.GPI : 0; P.gTA[v] = ok ? gg.TA : 0;
                    P.gcells[v] = ok ? gg.cells : 0; P.gstages[v] = ok ? gg.n_stages : 0;
                }
            }
            P.xq_off = off;
            off += ((((q.N + 3) >> 2) + 31) & ~31) * 16;       // 4 bytes per input; k-groups padded to 32 so that tails read zeros
        }
        bool shared = PH[ph].p[0].prologue == RWKV_PRO_LN_MIX && PH[ph].p[0].N <= 2 * kConsumers * 8;
        for (int z = 1; z < counts[ph] && shared; ++z)
            shared = PH[ph].p[z].prologue == RWKV_PRO_LN_MIX && PH[ph].p[z].share_ln && PH[ph].p[z].mode == PH[ph].p[0].mode &&
                     PH[ph].p[z].p2 == PH[ph].p[0].p2 && PH[ph].p[z].q0 == nullptr;
        PH[ph].ln_shared = shared ? 1 : 0;
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
