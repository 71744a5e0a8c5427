// Shared pieces of the mm8_one launch kernels (mm8_one.cu, mm8_cluster.cuh): problem descriptors,
// byte -> fp32 conversion, the fused prologues and epilogues, and the host-side launch planner.
#pragma once
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxRowsPerCta = 2048; // x' slice kept in shared memory
constexpr int kWideRowsPerCta = 2560; // the cluster kernel's second build: 20480 in-features (14B shape) / 8 splits
constexpr int kMaxSplit = 64;
constexpr int kPanelMin = 128;
constexpr int kCounterBytes = 4096;  // panel tickets (the last two words are unused)
constexpr int kMaxTickets = kCounterBytes / 4 - 2;
constexpr int kSumsBytes = (kCounterBytes / 4) * kMaxSplit * 4 * sizeof(float);  // [panel ticket][split][4]
constexpr int kMaxProblems = 4;
constexpr int kGroup = 4;            // rows drained per step
constexpr int ring_bytes(int depth) { return kGroup * depth * kThreads * 16; }   // 64 KB at depth 4

struct Problem {
    const void* x;
    const uint8_t* w;
    long long w_stride;
    const void* mx;
    const void* rx;
    const void* my;
    const void* ry;
    void* y;
    const void* aux;
    const void* aux2;
    int N, M;
    int epilogue;
    float out_scale;
    int prologue;
    // RWKV_PRO_LN_MIX: x is the residual stream; p0 = ln weight, p1 = ln bias, p2 = previous
    // token's LayerNorm output, p3 = mix vector, q0 = where this token's LayerNorm output goes
    // (may be NULL), mode = 0 (v4/v5 mix), 1 (v6 mix) or 2 (LayerNorm only).
    // RWKV_PRO_WKV4: x = r; p0 = k, p1 = v (fp16); f0 = t_decay, f1 = t_first, f2..f4 = aa, bb,
    // pp in; g0..g2 = aa, bb, pp out.
    const void *p0, *p1, *p2, *p3;
    void* q0;
    const float *f0, *f1, *f2, *f3, *f4;
    float *g0, *g1, *g2;
    int mode;
    int rows_per_cta;   // multiple of 32
    int splits;         // K-splits actually used by this problem
    long long partial_off;  // float offset of this problem's [splits][m_pad] block
    int m_pad;
    int counter_off;
};

struct Batch {
    Problem p[kMaxProblems];
    float* partial;
    float* sums;        // [panel ticket][kMaxSplit][4]
    unsigned* counters;
    int trace_id;       // launch number for the optional timeline below
};

// Optional per-CTA timeline for tuning (compiled in only with -DRWKV_MM8_TRACE): sixteen words per
// CTA per launch -- %globaltimer at entry, ring issued, predecessor done, prologue done, stream
// done, split reduction reached, exit; then the SM id.
#ifdef RWKV_MM8_TRACE
__device__ unsigned long long* g_mm8_trace = nullptr;
int g_mm8_trace_next = 0;       // host: launches so far
__device__ __forceinline__ void mm8_stamp(unsigned long long* row, int slot) {
    if (row != nullptr) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        if (slot == 7) { unsigned s; asm volatile("mov.u32 %0, %smid;" : "=r"(s)); t = s; }
        row[slot] = t;
    }
}
// the row pointer is fetched once, at entry: a stamp is then one posted store
#define MM8_TRACE_BEGIN(launch, cta)                                                                   \
    unsigned long long* mm8_tr = (threadIdx.x == 0 && g_mm8_trace != nullptr && (cta) < 1024)         \
                                     ? g_mm8_trace + ((long long)(launch) * 1024 + (cta)) * 16 : nullptr
#define MM8_STAMP(launch, cta, slot) mm8_stamp(mm8_tr, slot)
#else
#define MM8_TRACE_BEGIN(launch, cta) do { } while (0)
#define MM8_STAMP(launch, cta, slot) do { } while (0)
#endif

// byte i of `word` -> fp32 (2^23 + byte), then minus (2^23 + 128): exact (byte - 128).
__device__ __forceinline__ uint32_t code_bits(uint32_t word, int i) {
    return __byte_perm(word, 0x4B000000u, 0x7650 | i);
}
__device__ __forceinline__ float code(uint32_t word, int i) {
    return __uint_as_float(code_bits(word, i)) - 8388736.0f;
}

__device__ __forceinline__ uint4 ldg_bytes(const uint8_t* p, int valid) {
    uint32_t r[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i)
        if (i < valid) r[i >> 2] |= uint32_t(p[i]) << (8 * (i & 3));
    return make_uint4(r[0], r[1], r[2], r[3]);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_) : "memory"); }

// acc[16] += xv * (byte - 128) for the 16 bytes of v.  PACKED uses the two-wide fp32
// instructions of sm_100 (add.f32x2 / fma.rn.f32x2): 2 instead of 3 issue slots per byte.
template <bool PACKED>
__device__ __forceinline__ void fma16(float (&acc)[16], const uint4& v, float xv) {
    const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
    if (!PACKED) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[q * 4 + i] = fmaf(xv, code(wd[q], i), acc[q * 4 + i]);
    } else {
        unsigned long long x2, c2;
        asm("mov.b64 %0, {%1, %1};" : "=l"(x2) : "f"(xv));
        asm("mov.b64 %0, {%1, %1};" : "=l"(c2) : "f"(-8388736.0f));
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int i = 0; i < 4; i += 2) {
                unsigned long long f2, a2;
                asm("mov.b64 %0, {%1, %2};" : "=l"(f2) : "r"(code_bits(wd[q], i)), "r"(code_bits(wd[q], i + 1)));
                asm("mov.b64 %0, {%1, %2};" : "=l"(a2) : "f"(acc[q * 4 + i]), "f"(acc[q * 4 + i + 1]));
                asm("add.rn.f32x2 %0, %0, %1;" : "+l"(f2) : "l"(c2));
                asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(a2) : "l"(x2), "l"(f2));
                asm("mov.b64 {%0, %1}, %2;" : "=f"(acc[q * 4 + i]), "=f"(acc[q * 4 + i + 1]) : "l"(a2));
            }
    }
}

// Integer form of the same product: two rows at a time.  xq packs the two rows' activations as
// signed 16-bit fixed point (row a low, row b high); va / vb are the rows' 16 weight bytes.  Per
// word, two byte permutes interleave the rows ({a0 b0 a1 b1}, {a2 b2 a3 b3}) and four dp2a add
// xa*wa + xb*wb for one column each: 6 integer instructions for 8 bytes instead of 16 for the
// fp32 form.  acc[] are exact 32-bit sums of q*w with w the unsigned byte; the caller subtracts
// 128 times the sum of its q.
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
__device__ __forceinline__ void dot16_q(int (&acc)[16], const uint4& va, const uint4& vb, int xq) {
    const uint32_t wa[4] = {va.x, va.y, va.z, va.w};
    const uint32_t wb[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint32_t plo = __byte_perm(wa[q], wb[q], 0x5140);
        const uint32_t phi = __byte_perm(wa[q], wb[q], 0x7362);
        acc[q * 4 + 0] = dp2a_lo(xq, plo, acc[q * 4 + 0]);
        acc[q * 4 + 1] = dp2a_hi(xq, plo, acc[q * 4 + 1]);
        acc[q * 4 + 2] = dp2a_lo(xq, phi, acc[q * 4 + 2]);
        acc[q * 4 + 3] = dp2a_hi(xq, phi, acc[q * 4 + 3]);
    }
}

// Turn the CTA's x' (fp32, `nrows` values in xs) into packed 16-bit pairs IN PLACE: entry
// p * rpp + sub holds rows sub + 2p*rpp (low) and sub + (2p+1)*rpp (high), the two rows that the
// thread with row offset `sub` multiplies in its p-th pair; rows past nrows are 0.  `npairs` pairs
// per row offset (whole ring groups).  The thread with chunk index `ch` (of `cpr`) makes the pairs
// p = ch, ch + cpr, ... of its own row offset, at most NP of them.  Returns 1/scale (value = q /
// scale); the quantisation range is the largest that keeps a thread's 32-bit sums of `nsteps`
// products q * 255 from overflowing (32767 up to 257 steps).
template <int NP>   // pairs per thread at most: 8 up to 2048 rows per CTA, 10 up to 2560
__device__ __forceinline__ float quantize_pairs(float* xs, int rpp, int cpr, int sub, int ch, bool active,
                                                int npairs, int nsteps, int nrows, float m) {
    // m: the largest |x'| of the CTA's rows, +inf if any of them is not finite (the same in every thread)
    const int qmax = min(32767, 0x7fffffff / (255 * max(nsteps, 1)));
    const bool finite = m < 3.0e38f;            // false for inf and NaN
    const float scale = (finite && m > 0.f) ? float(qmax) / m : 0.f;
    float fa[NP], fb[NP];
#pragma unroll
    for (int i = 0; i < NP; ++i) {
        const int p = ch + i * cpr;
        fa[i] = fb[i] = 0.f;
        if (active && p < npairs) {
            const int ra = sub + 2 * p * rpp, rb = ra + rpp;
            if (ra < nrows) fa[i] = xs[ra];
            if (rb < nrows) fb[i] = xs[rb];
        }
    }
    __syncthreads();
    int* xp = reinterpret_cast<int*>(xs);
#pragma unroll
    for (int i = 0; i < NP; ++i) {
        const int p = ch + i * cpr;
        if (active && p < npairs) {
            const int qa = __float2int_rn(fa[i] * scale), qb = __float2int_rn(fb[i] * scale);
            xp[p * rpp + sub] = (qa & 0xffff) | (qb << 16);
        }
    }
    __syncthreads();
    if (!finite) return __int_as_float(0x7fc00000);      // non-finite activations: NaN results, as in fp32
    return m > 0.f ? m / float(qmax) : 0.f;
}

// Loads of activations and state go to L2 (ld.global.cg): under programmatic dependent launch they may
// have been written by another SM a moment ago, and L1 is not coherent.
template <typename F>
__device__ __forceinline__ float ldc(const void* base, int i) { return to_f32<F>(__ldcg(static_cast<const F*>(base) + i)); }

// Epilogue with the residual / multiplier operands already in hand (auxv = aux[k], aux2v = aux2[k]).
template <typename F>
__device__ __forceinline__ void store_epilogue_with(const Problem& P, int k, float val, float auxv, float aux2v) {
    switch (P.epilogue) {
    case RWKV_EPI_ACC_F32: {
        float* y = static_cast<float*>(P.y);
        y[k] = __ldcg(y + k) + val;
        break;
    }
    case RWKV_EPI_STORE:
        static_cast<F*>(P.y)[k] = from_f32<F>(val);
        break;
    case RWKV_EPI_SIGMOID: {
        float v = to_f32<F>(from_f32<F>(val));
        static_cast<F*>(P.y)[k] = from_f32<F>(1.0f / (1.0f + expf(-v)));
        break;
    }
    case RWKV_EPI_RELU_SQ: {
        float v = fmaxf(to_f32<F>(from_f32<F>(val)), 0.0f);
        static_cast<F*>(P.y)[k] = from_f32<F>(v * v);
        break;
    }
    case RWKV_EPI_RESIDUAL: {
        float v = to_f32<F>(from_f32<F>(val));
        float s = to_f32<F>(from_f32<F>(auxv + v));
        static_cast<F*>(P.y)[k] = from_f32<F>(s * P.out_scale);
        break;
    }
    case RWKV_EPI_MUL_RESIDUAL: {
        float v = to_f32<F>(from_f32<F>(val));
        float m = to_f32<F>(from_f32<F>(aux2v * v));
        float s = to_f32<F>(from_f32<F>(auxv + m));
        static_cast<F*>(P.y)[k] = from_f32<F>(s * P.out_scale);
        break;
    }
    case RWKV_EPI_STORE_F32:
        static_cast<float*>(P.y)[k] = to_f32<F>(from_f32<F>(val));
        break;
    case RWKV_EPI_SILU: {
        float v = to_f32<F>(from_f32<F>(val));
        static_cast<F*>(P.y)[k] = from_f32<F>(v / (1.0f + expf(-v)));
        break;
    }
    default: break;
    }
}

template <typename F>
__device__ __forceinline__ void store_epilogue(const Problem& P, int k, float val) {
    float auxv = 0.f, aux2v = 0.f;
    if (P.epilogue == RWKV_EPI_RESIDUAL || P.epilogue == RWKV_EPI_MUL_RESIDUAL) auxv = ldc<F>(P.aux, k);
    if (P.epilogue == RWKV_EPI_MUL_RESIDUAL) aux2v = ldc<F>(P.aux2, k);
    store_epilogue_with<F>(P, k, val, auxv, aux2v);
}

__device__ __forceinline__ float block_sum256(float v, float* sh8) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh8[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kWarps; ++i) t += sh8[i];
    return t;
}

// Copy n elements of ES bytes, starting at element `first` of `src_base`, to shared memory:
// 16-byte cp.async where the source is aligned (the caller commits), plain loads otherwise.
template <int ES>
__device__ __forceinline__ void stage_vec(uint8_t* dst, const void* src_base, int first, int n, int tid) {
    if (src_base == nullptr || n <= 0) return;
    const uint8_t* src = static_cast<const uint8_t*>(src_base) + (long long)first * ES;
    const int bytes = n * ES;
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        const int full = bytes >> 4;
        const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
        for (int c = tid; c < full; c += kThreads) cp_async16(d + c * 16, src + c * 16);
        done = full * 16;
    }
    for (int o = done + tid * ES; o < bytes; o += kThreads * ES) {
        if (ES == 2) *reinterpret_cast<uint16_t*>(dst + o) = __ldcg(reinterpret_cast<const uint16_t*>(src + o));
        else *reinterpret_cast<uint32_t*>(dst + o) = __ldcg(reinterpret_cast<const uint32_t*>(src + o));
    }
}

// Ask L2 for the lines of n elements of ES bytes from element `first` on (no data returns: the
// loads that follow the wait on the preceding kernel then find them on chip).
template <int ES>
__device__ __forceinline__ void l2_prefetch(const void* src_base, int first, int n, int tid) {
    if (src_base == nullptr || n <= 0) return;
    const uint8_t* src = static_cast<const uint8_t*>(src_base) + (long long)first * ES;
    const uint8_t* line0 = reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(src) & ~uintptr_t(127));
    const int lines = int((src + (long long)n * ES - line0 + 127) >> 7);
    for (int l = tid; l < lines; l += kThreads) asm volatile("prefetch.global.L2 [%0];" ::"l"(line0 + l * 128));
}

// The activation x[j] this problem multiplies with, for row j, after the fused prologue.
// LayerNorm statistics (mean, rstd) are computed once per CTA by the caller.
template <typename F>
__device__ __forceinline__ float prologue_value(const Problem& P, int j, float mean, float rstd, bool writer) {
    if (P.prologue == RWKV_PRO_PLAIN) return ldc<F>(P.x, j);
    if (P.prologue == RWKV_PRO_LN_MIX) {
        const float xx = r16((ldc<__half>(P.x, j) - mean) * rstd * __half2float(static_cast<const __half*>(P.p0)[j]) +
                             __half2float(static_cast<const __half*>(P.p1)[j]));
        if (writer && P.q0) static_cast<__half*>(P.q0)[j] = __float2half_rn(xx);
        if (P.mode == 2) return xx;
        const float sx = ldc<__half>(P.p2, j);
        const float mv = __half2float(static_cast<const __half*>(P.p3)[j]);
        if (P.mode == 0) return r16(r16(xx * mv) + r16(sx * r16(1.0f - mv)));
        return r16(xx + r16(r16(sx - xx) * mv));
    }
    // RWKV_PRO_WKV4 (pkg/model.py:1041-1055)
    const float r = ldc<__half>(P.x, j);
    const float kk = ldc<__half>(P.p0, j);
    const float vv = ldc<__half>(P.p1, j);
    const float a = __ldcg(P.f2 + j), b = __ldcg(P.f3 + j), p0 = __ldcg(P.f4 + j);
    float ww = P.f1[j] + kk;
    float p = fmaxf(p0, ww);
    float e1 = expf(p0 - p), e2 = expf(ww - p);
    const float wkv = r16((e1 * a + e2 * vv) / (e1 * b + e2));
    if (writer) {
        ww = P.f0[j] + p0;
        p = fmaxf(ww, kk);
        e1 = expf(ww - p); e2 = expf(kk - p);
        P.g0[j] = e1 * a + e2 * vv;
        P.g1[j] = e1 * b + e2;
        P.g2[j] = p;
    }
    return r16(r * wkv);
}


// ---------------------------------------------------------------------------------------------
// Host side: validate up to three problems and lay out one launch (panel width, K-splits,
// scratch offsets).  `slots` = CTAs that should run at once (CTAs per SM x SMs); `fit_only`
// forbids plans with more CTAs than slots.
// ---------------------------------------------------------------------------------------------
struct LaunchPlan {
    Batch b;
    int gx, gy, gz;     // grid: panels, splits, problems
    int pw;             // panel width in columns
    bool aligned;
};

static inline size_t mm8_ws_bytes_for(const int32_t* Ms, int count) {
    size_t bytes = size_t(kCounterBytes) + size_t(kSumsBytes);
    for (int i = 0; i < count; ++i) {
        int64_t m_pad = (int64_t(Ms[i]) + 511) / 512 * 512;
        bytes += size_t(kMaxSplit) * size_t(m_pad) * sizeof(float);
    }
    return bytes;
}

static inline size_t mm8_batch_ws_bytes(const rwkv_mm8_problem* problems, int count) {
    int32_t Ms[kMaxProblems] = {0, 0, 0, 0};
    for (int i = 0; i < count && i < kMaxProblems; ++i) Ms[i] = problems[i].M;
    return mm8_ws_bytes_for(Ms, count < kMaxProblems ? count : kMaxProblems);
}

static inline int mm8_plan(const rwkv_mm8_problem* problems, int count, int dtype, void* workspace,
                           size_t workspace_bytes, int slots, bool fit_only, int force_pw, int force_split,
                           const int* max_rows_by_prologue, LaunchPlan& plan) {
    RWKV_CHECK_ARG(problems != nullptr && count >= 1 && count <= kMaxProblems);
    RWKV_CHECK_ARG(dtype == RWKV_F16 || dtype == RWKV_F32);
    if (workspace == nullptr) return RWKV_ERR_WORKSPACE;
    RWKV_CHECK_ALIGN(workspace, 16);
    if (workspace_bytes < mm8_batch_ws_bytes(problems, count)) return RWKV_ERR_WORKSPACE;

    Batch& b = plan.b;
    b.counters = static_cast<unsigned*>(workspace);
    b.sums = reinterpret_cast<float*>(static_cast<char*>(workspace) + kCounterBytes);
    b.partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + kCounterBytes + kSumsBytes);

    bool aligned = true;
    long long total_cols = 0;
    for (int i = 0; i < count; ++i) {
        const rwkv_mm8_problem& q = problems[i];
        RWKV_CHECK_ARG(q.N >= 1 && q.M >= 1 && q.w_stride >= q.M);
        RWKV_CHECK_ARG(q.x && q.w && q.mx && q.rx && q.my && q.ry && q.y);
        RWKV_CHECK_ARG(q.epilogue >= RWKV_EPI_ACC_F32 && q.epilogue <= RWKV_EPI_SILU);
        if (q.epilogue == RWKV_EPI_RESIDUAL || q.epilogue == RWKV_EPI_MUL_RESIDUAL) RWKV_CHECK_ARG(q.aux != nullptr);
        if (q.epilogue == RWKV_EPI_MUL_RESIDUAL) RWKV_CHECK_ARG(q.aux2 != nullptr);
        RWKV_CHECK_ARG(q.prologue >= RWKV_PRO_PLAIN && q.prologue <= RWKV_PRO_WKV4);
        if (q.prologue == RWKV_PRO_LN_MIX) {
            RWKV_CHECK_ARG(dtype == RWKV_F16 && q.N <= 32 * kThreads && q.N % 8 == 0 && q.ln_w && q.ln_b &&
                           q.mode >= 0 && q.mode <= 2);
            RWKV_CHECK_ALIGN(q.x, 16);
            if (q.mode != 2) RWKV_CHECK_ARG(q.sx && q.mix);
        }
        if (q.prologue == RWKV_PRO_WKV4)
            RWKV_CHECK_ARG(dtype == RWKV_F16 && q.k && q.v && q.t_decay && q.t_first && q.aa && q.bb && q.pp &&
                           q.aa_out && q.bb_out && q.pp_out);
        const bool rows_padded = (q.M % 16 == 0) || (q.w_stride >= (q.M + 15) / 16 * 16);
        if (reinterpret_cast<uintptr_t>(q.w) % 16 != 0 || q.w_stride % 16 != 0 || !rows_padded) aligned = false;
        total_cols += q.M;
    }
    // Panel width: the widest of 512 / 256 / 128 columns that still gives enough panels for the
    // K-split count to stay small (the serial part of the split reduction grows with it).
    int pw = 512;
    if (force_pw != 0) pw = force_pw;
    else {
        while (pw > kPanelMin && (total_cols + pw - 1) / pw * 16 < slots) pw >>= 1;   // aim at <= 16 splits
    }
    int max_panels = 0, max_splits = 0;
    for (;; pw <<= 1) {         // fit_only: widen the panels until the tiles fit the slots
        int total_panels = 0;
        for (int i = 0; i < count; ++i) total_panels += (problems[i].M + pw - 1) / pw;
        if (total_panels > kMaxTickets) return RWKV_ERR_UNSUPPORTED;

        int counter_off = 0;
        max_panels = 0; max_splits = 0;
        long long partial_off = 0;
        const int rpp = kWarps * (512 / pw);       // rows per CTA step
        for (int i = 0; i < count; ++i) {
            const rwkv_mm8_problem& q = problems[i];
            Problem& P = b.p[i];
            P.x = q.x; P.w = q.w; P.w_stride = q.w_stride; P.mx = q.mx; P.rx = q.rx; P.my = q.my; P.ry = q.ry;
            P.y = q.y; P.aux = q.aux; P.aux2 = q.aux2; P.N = q.N; P.M = q.M; P.epilogue = q.epilogue;
            P.out_scale = q.out_scale;
            P.prologue = q.prologue; P.mode = q.mode;
            P.p0 = P.p1 = P.p2 = P.p3 = nullptr; P.q0 = nullptr;
            P.f0 = P.f1 = P.f2 = P.f3 = P.f4 = nullptr; P.g0 = P.g1 = P.g2 = nullptr;
            if (q.prologue == RWKV_PRO_LN_MIX) {
                P.p0 = q.ln_w; P.p1 = q.ln_b; P.p2 = q.sx; P.p3 = q.mix; P.q0 = q.xx_out;
            } else if (q.prologue == RWKV_PRO_WKV4) {
                P.p0 = q.k; P.p1 = q.v; P.f0 = q.t_decay; P.f1 = q.t_first; P.f2 = q.aa; P.f3 = q.bb; P.f4 = q.pp;
                P.g0 = q.aa_out; P.g1 = q.bb_out; P.g2 = q.pp_out;
            }
            const int panels = (q.M + pw - 1) / pw;
            const int max_rows = max_rows_by_prologue[q.prologue];
            int want = force_split > 0 ? force_split : slots / total_panels;
            // a grid that would leave more than 1/8 of the slots empty runs ~2.7 waves instead
            if (!fit_only && force_split == 0 && total_panels * want * 8 < slots * 7) want = (slots * 8 / 3) / total_panels;
            if (want < 1) want = 1;
            int min_split = (q.N + max_rows - 1) / max_rows;
            int max_split = (q.N + rpp - 1) / rpp;
            if (max_split > kMaxSplit) max_split = kMaxSplit;
            if (want > max_split) want = max_split;
            if (want < min_split) want = min_split;
            if (want > kMaxSplit) return RWKV_ERR_UNSUPPORTED;   // N beyond 64 * 2048 rows
            int rows = ((q.N + want - 1) / want + 31) / 32 * 32;
            if (rows > max_rows) rows = max_rows;
            P.rows_per_cta = rows;
            P.splits = (q.N + rows - 1) / rows;
            if (P.splits > kMaxSplit) return RWKV_ERR_UNSUPPORTED;
            P.m_pad = (q.M + 511) / 512 * 512;
            P.partial_off = partial_off;
            P.counter_off = counter_off;
            partial_off += (long long)kMaxSplit * P.m_pad;
            counter_off += panels;
            if (panels > max_panels) max_panels = panels;
            if (P.splits > max_splits) max_splits = P.splits;
        }

        if (!fit_only || pw >= 512 || force_pw != 0) break;
        long long tiles = 0;
        for (int i = 0; i < count; ++i) tiles += (long long)((problems[i].M + pw - 1) / pw) * b.p[i].splits;
        if (tiles <= slots) break;
    }
    for (int i = count; i < kMaxProblems; ++i) b.p[i] = b.p[0];
    plan.gx = max_panels; plan.gy = max_splits; plan.gz = count;
    plan.pw = pw;
    plan.aligned = aligned;
    return RWKV_OK;
}

}  // namespace
