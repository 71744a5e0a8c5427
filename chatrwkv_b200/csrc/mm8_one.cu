// mm8_one: decode-time dequantising GEMV, y[M] = x[N] @ dequant(W[N,M]).  HBM-bound: the
// only large operand is the uint8 matrix, read exactly once.
//
// Algebra (from the per-element form in the reference, pkg/cuda/operators.cu:224-228):
//   y[k] = rx[k] * sum_j (x[j]*ry[j]) * (w[j,k] - 128)            <- the streamed part
//        + rx[k] * 128.5 * sum_j x[j]*ry[j] + mx[k] * sum_j x[j] + sum_j x[j]*my[j]
// The byte codes are centred (w - 128) so the streamed sum does not cancel against the
// three scalar sums when x is one-signed (the FFN value matmul sees relu(k)^2 >= 0).
//
// Work split: grid = (column panels, K-splits, problems).  A CTA of 8 warps owns PW = 512,
// 256 or 128 columns x one contiguous slice of rows.  A thread owns 16 adjacent columns
// (one 16-byte chunk per row); PW/16 lanes cover a row, so a warp covers 1, 2 or 4 rows per
// step and the CTA 8, 16 or 32.
//
// Weight stream: every thread keeps a private ring of 16-byte slots in shared memory that
// it fills with cp.async (no registers held by loads in flight: 16 rows = 256 B per thread,
// 64 KB per CTA) and drains in groups of four.  Only the owning thread touches a slot, so
// the ring needs no barrier.
//
// Programmatic dependent launch: the kernel lets its successor start at once
// (launch_dependents) and fills its ring BEFORE waiting for its predecessor
// (griddepcontrol.wait): weights never depend on earlier kernels; everything else (x,
// state, the workspace) is touched only after the wait.
//
// Split-K: partial sums go through shared memory (CTA) and then through a global scratch
// buffer [split][column]; the last CTA to finish a panel (atomic ticket) adds the splits in
// split order, so the result does not depend on scheduling, and applies the epilogue.
//
// Prologues (what x is) and epilogues (what happens to y) fuse the pointwise neighbours of
// the matmuls in att_one / ffn_one (pkg/model.py:984-992, 1034-1055).
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxRowsPerCta = 2048; // x' slice kept in shared memory
constexpr int kMaxSplit = 64;
constexpr int kPanelMin = 128;
constexpr int kCounterBytes = 4096;  // 1024 panel tickets
constexpr int kSumsBytes = (kCounterBytes / 4) * kMaxSplit * 4 * sizeof(float);  // [panel ticket][split][4]
constexpr int kMaxProblems = 3;
constexpr int kGroup = 4;            // rows drained per step
constexpr int kDepth = 4;            // groups in flight
constexpr int kSlots = kGroup * kDepth;
constexpr int kRingBytes = kSlots * kThreads * 16;   // 64 KB

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
};

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

template <typename F>
__device__ __forceinline__ void store_epilogue(const Problem& P, int k, float val) {
    switch (P.epilogue) {
    case RWKV_EPI_ACC_F32: {
        float* y = static_cast<float*>(P.y);
        y[k] += val;
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
        float s = to_f32<F>(from_f32<F>(to_f32<F>(static_cast<const F*>(P.aux)[k]) + v));
        static_cast<F*>(P.y)[k] = from_f32<F>(s * P.out_scale);
        break;
    }
    case RWKV_EPI_MUL_RESIDUAL: {
        float v = to_f32<F>(from_f32<F>(val));
        float m = to_f32<F>(from_f32<F>(to_f32<F>(static_cast<const F*>(P.aux2)[k]) * v));
        float s = to_f32<F>(from_f32<F>(to_f32<F>(static_cast<const F*>(P.aux)[k]) + m));
        static_cast<F*>(P.y)[k] = from_f32<F>(s * P.out_scale);
        break;
    }
    case RWKV_EPI_STORE_F32:
        static_cast<float*>(P.y)[k] = to_f32<F>(from_f32<F>(val));
        break;
    default: break;
    }
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

// The activation x[j] this problem multiplies with, for row j, after the fused prologue.
// LayerNorm statistics (mean, rstd) are computed once per CTA by the caller.
template <typename F>
__device__ __forceinline__ float prologue_value(const Problem& P, int j, float mean, float rstd, bool writer) {
    if (P.prologue == RWKV_PRO_PLAIN) return to_f32<F>(static_cast<const F*>(P.x)[j]);
    if (P.prologue == RWKV_PRO_LN_MIX) {
        const __half* x = static_cast<const __half*>(P.x);
        const float xx = r16((__half2float(x[j]) - mean) * rstd * __half2float(static_cast<const __half*>(P.p0)[j]) +
                             __half2float(static_cast<const __half*>(P.p1)[j]));
        if (writer && P.q0) static_cast<__half*>(P.q0)[j] = __float2half_rn(xx);
        if (P.mode == 2) return xx;
        const float sx = __half2float(static_cast<const __half*>(P.p2)[j]);
        const float mv = __half2float(static_cast<const __half*>(P.p3)[j]);
        if (P.mode == 0) return r16(r16(xx * mv) + r16(sx * r16(1.0f - mv)));
        return r16(xx + r16(r16(sx - xx) * mv));
    }
    // RWKV_PRO_WKV4 (pkg/model.py:1041-1055)
    const float r = __half2float(static_cast<const __half*>(P.x)[j]);
    const float kk = __half2float(static_cast<const __half*>(P.p0)[j]);
    const float vv = __half2float(static_cast<const __half*>(P.p1)[j]);
    const float a = P.f2[j], b = P.f3[j], p0 = P.f4[j];
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

// LPR = lanes per row (PW / 16).  ALIGNED: cp.async ring; otherwise byte loads, any layout.
template <typename F, int LPR, bool ALIGNED, bool PACKED>
__global__ void __launch_bounds__(kThreads, 2) mm8_one_kernel(const __grid_constant__ Batch b) {
    asm volatile("griddepcontrol.launch_dependents;");
    constexpr int PW = LPR * 16;               // columns per CTA
    constexpr int RPW = 32 / LPR;              // rows per warp step
    constexpr int RPP = kWarps * RPW;          // rows per CTA step
    const Problem& P = b.p[blockIdx.z];
    const int panel = blockIdx.x;
    const int col0 = panel * PW;
    const int split = blockIdx.y;
    if (col0 >= P.M || split >= P.splits) return;

    extern __shared__ __align__(128) uint8_t ring[];    // [slot][thread] 16 B; later the reduce buffer
    __shared__ float xs[kMaxRowsPerCta];
    __shared__ float ssum[kWarps][3];
    __shared__ float sh8[kWarps];
    __shared__ unsigned s_ticket;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j0 = split * P.rows_per_cta;
    const int j1 = min(P.N, j0 + P.rows_per_cta);
    const int nrows = j1 - j0;
    const int sub = warp * RPW + lane / LPR;    // this thread's row within a CTA step
    const int c = col0 + (lane % LPR) * 16;
    const int valid = min(16, P.M - c);         // <= 0: this lane is past the last column
    const int nsteps = (nrows + RPP - 1) / RPP; // CTA steps; thread's row in step i is sub + i*RPP
    const int ngroups = (nsteps + kGroup - 1) / kGroup;
    const uint8_t* wp = P.w + (long long)(j0 + sub) * P.w_stride + c;
    const long long step = (long long)RPP * P.w_stride;
    const uint32_t slot0 = (uint32_t)__cvta_generic_to_shared(ring) + tid * 16;

    auto issue_group = [&](int g) {
        if (ALIGNED && valid > 0) {
#pragma unroll
            for (int u = 0; u < kGroup; ++u) {
                const int i = g * kGroup + u;
                if (sub + i * RPP < nrows) cp_async16(slot0 + ((g % kDepth) * kGroup + u) * (kThreads * 16), wp + i * step);
            }
        }
        cp_async_commit();
    };
    if (ALIGNED) {
#pragma unroll
        for (int g = 0; g < kDepth; ++g) issue_group(g);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- prologue: x for this CTA's rows, x' = x * ry, and this slice's scalar sums --------
    float mean = 0.f, rstd = 0.f;
    if (P.prologue == RWKV_PRO_LN_MIX) {
        const __half* x = static_cast<const __half*>(P.x);
        float v[32];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int d = tid + i * kThreads;
            v[i] = d < P.N ? __half2float(x[d]) : 0.f;
            s += v[i];
        }
        mean = block_sum256(s, sh8) / float(P.N);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const float d = (tid + i * kThreads) < P.N ? v[i] - mean : 0.f;
            q = fmaf(d, d, q);
        }
        rstd = rsqrtf(block_sum256(q, sh8) / float(P.N) + 1e-5f);
    }
    const F* ry = static_cast<const F*>(P.ry);
    const F* my = static_cast<const F*>(P.my);
    const bool writer = panel == 0;
    float sx = 0.f, sxr = 0.f, sxmy = 0.f;
    for (int j = j0 + tid; j < j1; j += kThreads) {
        const float xv = prologue_value<F>(P, j, mean, rstd, writer);
        const float xp = xv * to_f32<F>(ry[j]);
        xs[j - j0] = xp;
        sx += xv;
        sxr += xp;
        sxmy = fmaf(xv, to_f32<F>(my[j]), sxmy);
    }
    sx = warp_sum(sx); sxr = warp_sum(sxr); sxmy = warp_sum(sxmy);
    if (lane == 0) { ssum[warp][0] = sx; ssum[warp][1] = sxr; ssum[warp][2] = sxmy; }
    __syncthreads();

    // ---- main loop ---------------------------------------------------------------------------
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    if (ALIGNED) {
        for (int g = 0; g < ngroups; ++g) {
            cp_async_wait<kDepth - 1>();
            uint4 v[kGroup];
#pragma unroll
            for (int u = 0; u < kGroup; ++u)
                v[u] = *reinterpret_cast<const uint4*>(ring + tid * 16 + ((g % kDepth) * kGroup + u) * (kThreads * 16));
            if (valid > 0) {
#pragma unroll
                for (int u = 0; u < kGroup; ++u) {
                    const int r = sub + (g * kGroup + u) * RPP;
                    if (r < nrows) fma16<PACKED>(acc, v[u], xs[r]);
                }
            }
            issue_group(g + kDepth);            // refill the slots just consumed
        }
        cp_async_wait<0>();
    } else if (valid > 0) {
        for (int i = 0; sub + i * RPP < nrows; ++i) {
            const uint4 v = ldg_bytes(wp + i * step, valid);
            fma16<PACKED>(acc, v, xs[sub + i * RPP]);
        }
    }

    // ---- CTA reduce: (8 warps x RPW row groups) -> 1.  Element (lane % LPR, i) of row group rg
    // sits at position i*LPR + lane%LPR so that stores and loads are conflict free; position p
    // holds column (p % LPR) * 16 + p / LPR of the panel.
    __syncthreads();                             // every thread is done with its ring
    float* red = reinterpret_cast<float*>(ring);
    {
        const int rg = warp * RPW + lane / LPR, l = lane % LPR;
#pragma unroll
        for (int i = 0; i < 16; ++i) red[rg * PW + i * LPR + l] = acc[i];
    }
    __syncthreads();
    float* part = b.partial + P.partial_off + (long long)split * P.m_pad + col0;
    for (int p = tid; p < PW; p += kThreads) {
        float s = 0.f;
#pragma unroll
        for (int rg = 0; rg < RPP; ++rg) s += red[rg * PW + p];
        part[p] = s;
    }
    // This CTA's share of the scalar sums travels with its partials (same ticket).
    float* sums = b.sums + (long long)(P.counter_off + panel) * kMaxSplit * 4;
    if (tid < 3) {
        float s = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < kWarps; ++w8) s += ssum[w8][tid];
        sums[split * 4 + tid] = s;
    }

    // ---- ticket: the last CTA of this panel reduces over the splits -----------------------
    __threadfence();
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(&b.counters[P.counter_off + panel], 1u);
    __syncthreads();
    if (s_ticket != unsigned(P.splits - 1)) return;
    __threadfence();
    if (tid == 0) b.counters[P.counter_off + panel] = 0u;   // ready for the next call

    const int S = P.splits;
    // scalar sums: thread t < S fetches split t, then one block reduce per sum
    float t0 = 0.f, t1 = 0.f, t2 = 0.f;
    if (tid < S) {
        t0 = __ldcg(sums + tid * 4 + 0);
        t1 = __ldcg(sums + tid * 4 + 1);
        t2 = __ldcg(sums + tid * 4 + 2);
    }
    // partials: all loads of a thread are independent; 8 at a time
    constexpr int PPT = (PW + kThreads - 1) / kThreads;     // positions per thread (2, 1, 1)
    float sacc[PPT];
#pragma unroll
    for (int h = 0; h < PPT; ++h) sacc[h] = 0.f;
    const float* pbase = b.partial + P.partial_off + col0 + tid;
    const bool pos_ok = tid < PW;
    if (pos_ok) {
        int sp = 0;
        for (; sp + 8 <= S; sp += 8) {
            float a[8][PPT];
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
                for (int h = 0; h < PPT; ++h) a[u][h] = __ldcg(pbase + (long long)(sp + u) * P.m_pad + h * kThreads);
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
                for (int h = 0; h < PPT; ++h) sacc[h] += a[u][h];
        }
        for (; sp < S; ++sp)
#pragma unroll
            for (int h = 0; h < PPT; ++h) sacc[h] += __ldcg(pbase + (long long)sp * P.m_pad + h * kThreads);
    }
    const float tx = block_sum256(t0, sh8);
    const float txr = block_sum256(t1, sh8);
    const float txmy = block_sum256(t2, sh8);

    const F* mx = static_cast<const F*>(P.mx);
    const F* rx = static_cast<const F*>(P.rx);
#pragma unroll
    for (int h = 0; h < PPT; ++h) {
        const int p = tid + h * kThreads;
        const int k = col0 + (p % LPR) * 16 + p / LPR;
        if (p < PW && k < P.M) {
            const float rxk = to_f32<F>(rx[k]);
            const float val = fmaf(rxk, sacc[h], fmaf(rxk * 128.5f, txr, fmaf(to_f32<F>(mx[k]), tx, txmy)));
            store_epilogue<F>(P, k, val);
        }
    }
}

int g_split_override = 0;
int g_variant = 0;

}  // namespace

extern "C" void rwkv_mm8_one_set_split(int split) { g_split_override = split; }
// bits 0-1: panel width (0 = automatic, 1 = 512, 2 = 256, 3 = 128 columns); bit 2: scalar fp32
// arithmetic instead of the two-wide instructions
extern "C" void rwkv_mm8_one_set_variant(int variant) { g_variant = variant; }

static size_t ws_bytes_for(const int32_t* Ms, int count) {
    size_t bytes = size_t(kCounterBytes) + size_t(kSumsBytes);
    for (int i = 0; i < count; ++i) {
        int64_t m_pad = (int64_t(Ms[i]) + 511) / 512 * 512;
        bytes += size_t(kMaxSplit) * size_t(m_pad) * sizeof(float);
    }
    return bytes;
}

extern "C" size_t rwkv_mm8_one_workspace_bytes(int64_t N, int64_t M) {
    (void)N;
    int32_t m = int32_t(M);
    return ws_bytes_for(&m, 1);
}

extern "C" size_t rwkv_mm8_one_batch_workspace_bytes(const rwkv_mm8_problem* problems, int count) {
    int32_t Ms[kMaxProblems] = {0, 0, 0};
    for (int i = 0; i < count && i < kMaxProblems; ++i) Ms[i] = problems[i].M;
    return ws_bytes_for(Ms, count < kMaxProblems ? count : kMaxProblems);
}

extern "C" int rwkv_mm8_one_batch(const rwkv_mm8_problem* problems, int count, int dtype,
                                  void* workspace, size_t workspace_bytes, void* stream) {
    RWKV_CHECK_ARG(problems != nullptr && count >= 1 && count <= kMaxProblems);
    RWKV_CHECK_ARG(dtype == RWKV_F16 || dtype == RWKV_F32);
    if (workspace == nullptr) return RWKV_ERR_WORKSPACE;
    RWKV_CHECK_ALIGN(workspace, 16);
    if (workspace_bytes < rwkv_mm8_one_batch_workspace_bytes(problems, count)) return RWKV_ERR_WORKSPACE;

    Batch b;
    b.counters = static_cast<unsigned*>(workspace);
    b.sums = reinterpret_cast<float*>(static_cast<char*>(workspace) + kCounterBytes);
    b.partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + kCounterBytes + kSumsBytes);

    bool aligned = true;
    long long total_cols = 0;
    for (int i = 0; i < count; ++i) {
        const rwkv_mm8_problem& q = problems[i];
        RWKV_CHECK_ARG(q.N >= 1 && q.M >= 1 && q.w_stride >= q.M);
        RWKV_CHECK_ARG(q.x && q.w && q.mx && q.rx && q.my && q.ry && q.y);
        RWKV_CHECK_ARG(q.epilogue >= RWKV_EPI_ACC_F32 && q.epilogue <= RWKV_EPI_STORE_F32);
        if (q.epilogue == RWKV_EPI_RESIDUAL || q.epilogue == RWKV_EPI_MUL_RESIDUAL) RWKV_CHECK_ARG(q.aux != nullptr);
        if (q.epilogue == RWKV_EPI_MUL_RESIDUAL) RWKV_CHECK_ARG(q.aux2 != nullptr);
        RWKV_CHECK_ARG(q.prologue >= RWKV_PRO_PLAIN && q.prologue <= RWKV_PRO_WKV4);
        if (q.prologue == RWKV_PRO_LN_MIX) {
            RWKV_CHECK_ARG(dtype == RWKV_F16 && q.N <= 32 * kThreads && q.ln_w && q.ln_b && q.mode >= 0 && q.mode <= 2);
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
    const int sms = rwkv_sm_count();
    const int slots = 2 * sms;
    int pw = 512;
    if ((g_variant & 3) != 0) pw = 1024 >> (g_variant & 3);
    else {
        while (pw > kPanelMin && (total_cols + pw - 1) / pw * 16 < slots) pw >>= 1;   // aim at <= 16 splits
    }
    int total_panels = 0;
    for (int i = 0; i < count; ++i) total_panels += (problems[i].M + pw - 1) / pw;
    if (total_panels > kCounterBytes / 4) return RWKV_ERR_UNSUPPORTED;

    int max_panels = 0, max_splits = 0, counter_off = 0;
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
        int want = g_split_override > 0 ? g_split_override : slots / total_panels;
        if (g_split_override == 0 && total_panels * want * 8 < slots * 7) want = (slots * 8 / 3) / total_panels;   // poor fit: ~2.7 waves
        if (want < 1) want = 1;
        int min_split = (q.N + kMaxRowsPerCta - 1) / kMaxRowsPerCta;
        int max_split = (q.N + rpp - 1) / rpp;
        if (max_split > kMaxSplit) max_split = kMaxSplit;
        if (want > max_split) want = max_split;
        if (want < min_split) want = min_split;
        if (want > kMaxSplit) return RWKV_ERR_UNSUPPORTED;   // N beyond 64 * 2048 rows
        int rows = ((q.N + want - 1) / want + 31) / 32 * 32;
        if (rows > kMaxRowsPerCta) rows = kMaxRowsPerCta;
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
    for (int i = count; i < kMaxProblems; ++i) b.p[i] = b.p[0];

    dim3 grid(max_panels, max_splits, count);
    const bool packed = (g_variant & 4) == 0;
    void (*kern)(Batch) = nullptr;
#define RWKV_PICK(FT)                                                                                        \
    if (!aligned) kern = pw == 512 ? mm8_one_kernel<FT, 32, false, false>                                   \
                       : pw == 256 ? mm8_one_kernel<FT, 16, false, false> : mm8_one_kernel<FT, 8, false, false>; \
    else if (packed) kern = pw == 512 ? mm8_one_kernel<FT, 32, true, true>                                  \
                          : pw == 256 ? mm8_one_kernel<FT, 16, true, true> : mm8_one_kernel<FT, 8, true, true>; \
    else kern = pw == 512 ? mm8_one_kernel<FT, 32, true, false>                                             \
              : pw == 256 ? mm8_one_kernel<FT, 16, true, false> : mm8_one_kernel<FT, 8, true, false>;
    if (dtype == RWKV_F16) { RWKV_PICK(__half) } else { RWKV_PICK(float) }
#undef RWKV_PICK
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes) != cudaSuccess) {
        cudaGetLastError();
        return RWKV_ERR_LAUNCH;
    }
    return rwkv_launch_pdl(kern, grid, dim3(kThreads), size_t(kRingBytes), static_cast<cudaStream_t>(stream), b);
}

extern "C" int rwkv_mm8_one(int64_t N, int64_t M, const void* x, const uint8_t* w, int64_t w_stride,
                            const void* mx, const void* rx, const void* my, const void* ry, int dtype,
                            float* y, void* workspace, size_t workspace_bytes, void* stream) {
    RWKV_CHECK_ARG(N >= 1 && M >= 1 && N <= INT32_MAX && M <= INT32_MAX);
    rwkv_mm8_problem q = {};
    q.x = x; q.w = w; q.w_stride = w_stride; q.mx = mx; q.rx = rx; q.my = my; q.ry = ry;
    q.y = y; q.N = int32_t(N); q.M = int32_t(M);
    q.epilogue = RWKV_EPI_ACC_F32; q.out_scale = 1.0f; q.prologue = RWKV_PRO_PLAIN;
    return rwkv_mm8_one_batch(&q, 1, dtype, workspace, workspace_bytes, stream);
}

// ---------------------------------------------------------------------------------------------
// mm8_one for callers that cannot allocate device memory.
//
// Same kernel, same split plan and the same result as rwkv_mm8_one, but the split-K scratch
// (panel tickets, per-split scalar sums, per-split partial rows) lives in one fixed array in
// the library's own device image instead of a caller-provided workspace.  The array costs
// kStaticScratchBytes (about 9 MiB) on every GPU that loads the library, for as long as the
// process lives, and bounds the out-feature count at kStaticMaxM.
//
// `g_static_scratch` names a DEVICE symbol.  In host code that name is only a stand-in: the
// address a kernel may use comes from cudaGetSymbolAddress, looked up once per device (with
// that device current) on the first call and remembered in g_static_ptr[].
// ---------------------------------------------------------------------------------------------
namespace {
constexpr int kStaticMaxM = 32768;
constexpr size_t kStaticScratchBytes =
    size_t(kCounterBytes) + size_t(kSumsBytes) + size_t(kMaxSplit) * size_t(kStaticMaxM) * sizeof(float);
constexpr int kStaticMaxDevices = 64;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
void* g_static_ptr[kStaticMaxDevices] = {};
}  // namespace

extern "C" int rwkv_mm8_one_static(int64_t N, int64_t M, const void* x, const uint8_t* w, int64_t w_stride,
                                   const void* mx, const void* rx, const void* my, const void* ry, int dtype,
                                   float* y, void* stream) {
    RWKV_CHECK_ARG(N >= 1 && M >= 1 && N <= INT32_MAX);
    if (M > kStaticMaxM) return RWKV_ERR_STATIC_LIMIT;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) {
        cudaGetLastError();
        return RWKV_ERR_LAUNCH;
    }
    if (g_static_ptr[dev] == nullptr) {
        // First call on this device: resolve the symbol to this device's copy of the array.
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
            cudaGetLastError();
            return RWKV_ERR_LAUNCH;
        }
        g_static_ptr[dev] = p;
    }
    // The tickets must read zero when the kernel starts.  Every finished call leaves them so;
    // clearing them here as well makes the call independent of how an earlier one ended.
    if (cudaMemsetAsync(g_static_ptr[dev], 0, kCounterBytes, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        cudaGetLastError();
        return RWKV_ERR_LAUNCH;
    }
    return rwkv_mm8_one(N, M, x, w, w_stride, mx, rx, my, ry, dtype, y, g_static_ptr[dev], kStaticScratchBytes, stream);
}
