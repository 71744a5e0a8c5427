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
#include "mm8_core.cuh"
#include "mm8_lean.cuh"

namespace {

// LPR = lanes per row (PW / 16).  ALIGNED: cp.async ring; otherwise byte loads, any layout.
template <typename F, int LPR, bool ALIGNED, bool PACKED, int kDepth>
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
    const int cta_id = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    (void)cta_id;
    MM8_TRACE_BEGIN(b.trace_id, cta_id);
    MM8_STAMP(b.trace_id, cta_id, 0);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    MM8_STAMP(b.trace_id, cta_id, 2);

    // ---- prologue: x for this CTA's rows, x' = x * ry, and this slice's scalar sums --------
    float mean = 0.f, rstd = 0.f;
    if (P.prologue == RWKV_PRO_LN_MIX) {
        // The whole vector in registers: up to four 16-byte loads per thread, issued together.
        const __half* x = static_cast<const __half*>(P.x);
        const int nvec = P.N / 8;               // host guarantees N % 8 == 0 and N <= 8192
        uint4 xv4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int v = tid + i * kThreads;
            xv4[i] = v < nvec ? __ldcg(reinterpret_cast<const uint4*>(x) + v) : make_uint4(0, 0, 0, 0);
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2* h = reinterpret_cast<const __half2*>(&xv4[i]);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h[e]); s += f.x + f.y; }
        }
        mean = block_sum256(s, sh8) / float(P.N);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (tid + i * kThreads < nvec) {
                const __half2* h = reinterpret_cast<const __half2*>(&xv4[i]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h[e]);
                    q = fmaf(f.x - mean, f.x - mean, q);
                    q = fmaf(f.y - mean, f.y - mean, q);
                }
            }
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
    MM8_STAMP(b.trace_id, cta_id, 3);

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

    MM8_STAMP(b.trace_id, cta_id, 4);
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
    MM8_STAMP(b.trace_id, cta_id, 5);
    MM8_STAMP(b.trace_id, cta_id, 7);
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
    MM8_STAMP(b.trace_id, cta_id, 6);
}

int g_split_override = 0;
int g_variant = 0;

}  // namespace

extern "C" void rwkv_mm8_one_set_split(int split) { g_split_override = split; }
// bits 0-1: panel width (0 = automatic, 1 = 512, 2 = 256, 3 = 128 columns); bit 2: scalar fp32
// arithmetic; bit 3: two-wide fp32 arithmetic in the cluster kernel (its default is the 16-bit
// fixed-point form)
extern "C" void rwkv_mm8_one_set_variant(int variant) { g_variant = variant; }

extern "C" size_t rwkv_mm8_one_workspace_bytes(int64_t N, int64_t M) {
    (void)N;
    int32_t m = int32_t(M);
    return mm8_ws_bytes_for(&m, 1);
}

#ifdef RWKV_MM8_TRACE
// tuning builds only: where the per-CTA timeline goes ([launch][1024 CTAs][16] words); restarts the launch count
extern "C" int rwkv_mm8_trace_set(unsigned long long* buffer) {
    g_mm8_trace_next = 0;
    return cudaMemcpyToSymbol(g_mm8_trace, &buffer, sizeof(buffer)) == cudaSuccess ? RWKV_OK : RWKV_ERR_LAUNCH;
}
#endif

extern "C" void rwkv_mm8_one_set_lean(int on) { g_use_lean = on < 0 ? -1 : (on != 0); }

extern "C" int rwkv_mm8_one_take_error(void* stream, int* error) {
    RWKV_CHECK_ARG(error != nullptr);
    unsigned* word = lean_error_word();
    if (word == nullptr) return RWKV_ERR_LAUNCH;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned v = 0;
    if (cudaMemcpyAsync(&v, word, sizeof(v), cudaMemcpyDeviceToHost, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess) {
        cudaGetLastError();
        return RWKV_ERR_LAUNCH;
    }
    if (v != 0 && cudaMemsetAsync(word, 0, sizeof(v), st) != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    *error = int(v);
    return RWKV_OK;
}

extern "C" size_t rwkv_mm8_one_batch_workspace_bytes(const rwkv_mm8_problem* problems, int count) {
    return mm8_batch_ws_bytes(problems, count);
}

static int mm8_one_batch_impl(const rwkv_mm8_problem* problems, int count, const rwkv_mm8_exchange* exchange, int dtype,
                              int flags, void* workspace, size_t workspace_bytes, void* stream);

extern "C" int rwkv_mm8_one_batch(const rwkv_mm8_problem* problems, int count, int dtype,
                                  void* workspace, size_t workspace_bytes, void* stream) {
    return mm8_one_batch_impl(problems, count, nullptr, dtype, 0, workspace, workspace_bytes, stream);
}

extern "C" int rwkv_mm8_one_batch_exchange(const rwkv_mm8_problem* problems, int count, const rwkv_mm8_exchange* exchange,
                                           int dtype, void* workspace, size_t workspace_bytes, void* stream) {
    return mm8_one_batch_impl(problems, count, exchange, dtype, 0, workspace, workspace_bytes, stream);
}

extern "C" int rwkv_mm8_one_batch_flags(const rwkv_mm8_problem* problems, int count, const rwkv_mm8_exchange* exchange,
                                        int dtype, int flags, void* workspace, size_t workspace_bytes, void* stream) {
    return mm8_one_batch_impl(problems, count, exchange, dtype, flags, workspace, workspace_bytes, stream);
}

static int mm8_one_batch_impl(const rwkv_mm8_problem* problems, int count, const rwkv_mm8_exchange* exchange, int dtype,
                              int flags, void* workspace, size_t workspace_bytes, void* stream) {
    LaunchPlan plan;
    static const int max_rows[3] = {kMaxRowsPerCta, kMaxRowsPerCta, kMaxRowsPerCta};
    const int force_pw = (g_variant & 3) != 0 ? (1024 >> (g_variant & 3)) : 0;
    const int rc = mm8_plan(problems, count, dtype, workspace, workspace_bytes, 2 * rwkv_sm_count(), false,
                            force_pw, g_split_override, max_rows, plan);
    if (rc != RWKV_OK) return rc;
    const int pw = plan.pw;
    const bool aligned = plan.aligned, packed = (g_variant & 4) == 0;
    Exchange ex;
    const Exchange* exp = nullptr;
    if (exchange != nullptr) {
        // results also go to the other ranks; only the cluster kernel does that
        const rwkv_mm8_exchange& q = *exchange;
        RWKV_CHECK_ARG(q.world >= 2 && q.world <= 8 && q.rank >= 0 && q.rank < q.world);
        RWKV_CHECK_ARG(q.arrived && q.done_counter && q.error && q.signal_seq != 0);
        memset(&ex, 0, sizeof(ex));
        ex.n_peers = q.world - 1;
        for (int pr = 0; pr < ex.n_peers; ++pr) {
            RWKV_CHECK_ARG(q.peer_arrived[pr] != nullptr);
            ex.peer_arrived[pr] = q.peer_arrived[pr];
            for (int z = 0; z < count; ++z) {
                RWKV_CHECK_ARG(q.peer_y[z][pr] != nullptr && problems[z].epilogue != RWKV_EPI_ACC_F32);
                ex.peer_y[z][pr] = q.peer_y[z][pr];
            }
        }
        ex.arrived = q.arrived; ex.done_counter = q.done_counter; ex.error = q.error;
        ex.seq_base = q.seq_base;
        ex.wait_seq = q.wait_seq; ex.signal_seq = q.signal_seq; ex.world = q.world; ex.rank = q.rank;
        exp = &ex;
    }
    if (aligned && (g_variant & 3) == 0 && g_split_override == 0) {
        // K-splits of a panel as one thread-block cluster (mm8_cluster.cuh); falls through to the
        // ticket kernel when the batch is not eligible.
        if (exp == nullptr && dtype == RWKV_F16 && (g_variant & 12) == 0) {
            const int lrc = mm8_lean_launch(plan.b, count, (flags & RWKV_MM8_WIDE_BUILD) != 0, static_cast<cudaStream_t>(stream));
            if (lrc != RWKV_ERR_UNSUPPORTED) return lrc;
        }
        const int crc = mm8_cluster_launch(plan.b, count, dtype, (g_variant & 4) ? 0 : (g_variant & 8) ? 1 : 2, exp, (flags & RWKV_MM8_WIDE_BUILD) != 0,
                                           static_cast<cudaStream_t>(stream));
        if (crc != RWKV_ERR_UNSUPPORTED) return crc;
    }
    if (exp != nullptr) return RWKV_ERR_UNSUPPORTED;
    void (*kern)(Batch) = nullptr;
#define RWKV_PICK(FT)                                                                                        \
    if (!aligned) kern = pw == 512 ? mm8_one_kernel<FT, 32, false, false, 4>                                \
                       : pw == 256 ? mm8_one_kernel<FT, 16, false, false, 4> : mm8_one_kernel<FT, 8, false, false, 4>; \
    else if (packed) kern = pw == 512 ? mm8_one_kernel<FT, 32, true, true, 4>                               \
                          : pw == 256 ? mm8_one_kernel<FT, 16, true, true, 4> : mm8_one_kernel<FT, 8, true, true, 4>; \
    else kern = pw == 512 ? mm8_one_kernel<FT, 32, true, false, 4>                                          \
              : pw == 256 ? mm8_one_kernel<FT, 16, true, false, 4> : mm8_one_kernel<FT, 8, true, false, 4>;
    if (dtype == RWKV_F16) { RWKV_PICK(__half) } else { RWKV_PICK(float) }
#undef RWKV_PICK
    // The ring needs 64 KB; asking for 104 KB caps residency at two CTAs per SM.  With room for
    // a third, the block scheduler packs a one-wave grid onto fewer SMs and the launch slows
    // down (measured: 341 instead of 410 tokens/s at the 7B shape).
    const int smem = 104 * 1024;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
        cudaGetLastError();
        return RWKV_ERR_LAUNCH;
    }
    plan.b.trace_id = 0;
#ifdef RWKV_MM8_TRACE
    plan.b.trace_id = g_mm8_trace_next++;
#endif
    return rwkv_launch_pdl(kern, dim3(plan.gx, plan.gy, plan.gz), dim3(kThreads), size_t(smem),
                           static_cast<cudaStream_t>(stream), plan.b);
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
// that device current) on the first call and remembered in g_static_ptr[] (filled without a
// lock: like the tuning hooks, not thread-safe -- make the first call per device from one thread).
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
