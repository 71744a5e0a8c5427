// mm8_one for the decode step, cut down to the instructions a launch cannot do without.
//
// A decode token is ~130 dependent launches of 10-15 us, and per-CTA timelines of mm8_cluster_kernel
// showed ~7 us of every launch going to code that runs once per CTA -- staging constants, LayerNorm,
// quantising x', the split-K reduction -- at 5-8 clocks per instruction (two warps per scheduler, every
// instruction waiting for the one before it), with the HBM idle meanwhile.  This kernel keeps the stream
// loop of mm8_cluster_kernel (per-thread cp.async ring, 16-bit fixed-point x', dp2a) and rewrites what
// surrounds it for the common decode case (fp16 activations, integer arithmetic, slices that fit the
// staging areas, one GPU):
//   * model constants and the previous token's state reach shared memory by bulk copies that ONE thread
//     issues before the wait on the preceding kernel (a dozen instructions instead of seven copy loops);
//   * the rows of a CTA are dealt to ALL its threads after one pass of LayerNorm statistics, so the
//     pointwise chain per thread is 2-4 rows long instead of 8 on a quarter of the threads;
//   * x' goes from registers straight to its 16-bit place (no fp32 round trip through shared memory);
//   * every CTA PUSHES its column sums into the shared memory of the CTA that finishes those columns
//     (remote stores), so one cluster barrier replaces barrier + remote loads + barrier, and a CTA
//     leaves as soon as its own columns are stored;
//   * index arithmetic by multiply-high with reciprocals that the host tabulates for full-width panels.
// The integer dot products are exact as in mm8_cluster_kernel and the split-K sums are added in the same rank
// order; results differ from that kernel's by the order of a few fp32 additions (the scalar sums of x, the row
// groups of a panel of another width) and by the LayerNorm statistics, taken in one pass around x[0] instead of
// two passes: ulps of fp32 before the fp16 rounding.  Two runs of this kernel are bit-identical.  Launches that
// do not qualify go to mm8_cluster_kernel.
#pragma once
#include "mm8_cluster.cuh"

namespace {

constexpr int kLeanExtraBytes = 24 * 1024;       // LN: ln w, ln b, mix, previous x, this x (2 KB each); WKV: 5 x 4 KB
constexpr int kLeanExtraRows = 1024;             // rows per CTA that the LayerNorm / WKV prologues can stage
template <int ROWS> constexpr int lean_stage_bytes() { return 2 * ROWS * 2 + kLeanExtraBytes + 2 * kStageEpiCols * 2; }

struct LeanBatch {
    Problem p[kMaxProblems];
    int panel_start[kMaxProblems + 1];
    int pw, S, s_log2, trace_id;
    int cpr, rpp;                    // of a full-width panel
    unsigned m_cpr, m_rpp;           // ceil(2^32 / cpr), ceil(2^32 / rpp) (0 stands for 2^32: divisor 1)
    unsigned* error;                 // set to 1 when a bounded wait gives up
};

__device__ unsigned g_lean_error = 0;
int g_use_lean = -1;             // -1 = the environment decides (RWKV_B200_LEAN=0 turns it off), else 0 / 1

__device__ __forceinline__ int fast_div(int n, int d, unsigned m) { return d == 1 ? n : int(__umulhi(unsigned(n), m)); }
__device__ __forceinline__ uint32_t lean_s2u(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lean_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void lean_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool lean_mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void lean_bulk(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void st_remote_f32(uint32_t local_addr, uint32_t cta_rank, float v) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta_rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(r), "f"(v) : "memory");
}

template <int ROWS>
__global__ void __launch_bounds__(kThreads, 2) mm8_lean_kernel(const __grid_constant__ LeanBatch b) {
    using F = __half;
    asm volatile("griddepcontrol.launch_dependents;");
    MM8_TRACE_BEGIN(b.trace_id, blockIdx.x);
    MM8_STAMP(b.trace_id, blockIdx.x, 1);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int S = b.S;
    const int rank = int(blockIdx.x) & (S - 1);          // == %cluster_ctarank for clusters along x
    const int cid = int(blockIdx.x) >> b.s_log2;
    int z = 0;
#pragma unroll
    for (int i = 1; i < kMaxProblems; ++i) z += cid >= b.panel_start[i] ? 1 : 0;
    const Problem& P = b.p[z];
    const int panel = cid - b.panel_start[z];
    const int col0 = panel * b.pw;
    const int ncols = min(b.pw, P.M - col0);             // >= 1 by construction of the grid
    int cpr = b.cpr, rpp = b.rpp;
    unsigned m_cpr = b.m_cpr, m_rpp = b.m_rpp;
    if (ncols != b.pw) {                                 // the narrower last panel of a matrix
        cpr = (ncols + 15) >> 4;
        rpp = kThreads / cpr;
        m_cpr = 0xffffffffu / unsigned(cpr) + 1u;
        m_rpp = 0xffffffffu / unsigned(rpp) + 1u;
    }
    const int PWc = cpr * 16;
    const int j0 = rank * P.rows_per_cta;                // rows_per_cta is a multiple of 8
    const int j1 = min(P.N, j0 + P.rows_per_cta);
    const int nrows = max(0, j1 - j0);                   // a multiple of 8 (the host checks N % 8 == 0)
    const int sub = fast_div(tid, cpr, m_cpr);           // this thread's row within a CTA step
    const int ch = tid - sub * cpr;                      // this thread's 16-byte chunk within the row
    const bool active = sub < rpp;
    const int nsteps = fast_div(nrows + rpp - 1, rpp, m_rpp);
    const int ngroups = (nsteps + kGroup - 1) / kGroup;
    // columns this CTA finishes after the cluster reduction: [kc0, kc1) of the panel
    const int per = (((ncols + S - 1) >> b.s_log2) + 7) & ~7;
    const int kc0 = min(ncols, rank * per), kc1 = min(ncols, kc0 + per);

    extern __shared__ __align__(128) uint8_t ring[];     // [slot][thread] 16 B; later the CTA's reduce buffer
    static_assert(ring_bytes(kDepthC) + lean_stage_bytes<ROWS>() <= cluster_smem<ROWS>(), "stage area does not fit");
    __shared__ int xs[ROWS];                             // x' as pairs of 16-bit fixed point
    __shared__ float ssum[kWarps][4];                    // per warp: sum x, sum x', sum x my, largest |x'|
    __shared__ float sh8[2 * kWarps];
    __shared__ float gat3[kMaxClusterSize][4];           // every rank's scalar sums (pushed by the ranks)
    __shared__ __align__(8) unsigned long long mbar;

    uint8_t* stage = ring + ring_bytes(kDepthC);
    F* s_ry = reinterpret_cast<F*>(stage);
    F* s_my = s_ry + ROWS;
    uint8_t* s_extra = stage + 2 * ROWS * sizeof(F);
    F* s_rx = reinterpret_cast<F*>(s_extra + kLeanExtraBytes);
    F* s_mx = s_rx + kStageEpiCols;
    float* gather = reinterpret_cast<float*>(stage);     // [S][per] after the prologue: the ranks' sums of MY columns
    const int ncol8 = (kc1 - kc0) & ~7;                  // columns whose rx, mx come by bulk copy
    // divisions that the code after the wait would otherwise pay for
    const unsigned m_per = 0xffffffffu / unsigned(per) + 1u;            // per >= 8
    const int qmax = min(32767, 0x7fffffff / (255 * max(nsteps, 1)));   // see the quantisation below
    const float invn = 1.0f / float(P.N);
    const int cnt = (active && sub < nrows) ? fast_div(nrows - sub + rpp - 1, rpp, m_rpp) : 0;     // rows of this thread

    // ---- before the preceding kernel is known to be done: model constants and last token's state ----
    if (tid == 0) {
        lean_mbar_init(lean_s2u(&mbar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid == kThreads - 32) {
        const uint32_t bar = lean_s2u(&mbar);
        const uint32_t rb = uint32_t(nrows) * 2u, cbytes = uint32_t(ncol8) * 2u;
        uint32_t total = 2u * rb + 2u * cbytes;
        if (P.prologue == RWKV_PRO_LN_MIX) total += 2u * rb + (P.mode != 2 ? 2u * rb : 0u);
        else if (P.prologue == RWKV_PRO_WKV4) total += 10u * rb;
        lean_mbar_expect_tx(bar, total);
        if (rb) {
            lean_bulk(lean_s2u(s_ry), static_cast<const F*>(P.ry) + j0, rb, bar);
            lean_bulk(lean_s2u(s_my), static_cast<const F*>(P.my) + j0, rb, bar);
            if (P.prologue == RWKV_PRO_LN_MIX) {
                lean_bulk(lean_s2u(s_extra), static_cast<const F*>(P.p0) + j0, rb, bar);                // ln weight
                lean_bulk(lean_s2u(s_extra + 2048), static_cast<const F*>(P.p1) + j0, rb, bar);         // ln bias
                if (P.mode != 2) {
                    lean_bulk(lean_s2u(s_extra + 4096), static_cast<const F*>(P.p3) + j0, rb, bar);     // mix
                    lean_bulk(lean_s2u(s_extra + 6144), static_cast<const F*>(P.p2) + j0, rb, bar);     // previous token's x
                }
            } else if (P.prologue == RWKV_PRO_WKV4) {
                lean_bulk(lean_s2u(s_extra), P.f0 + j0, 2u * rb, bar);             // t_decay
                lean_bulk(lean_s2u(s_extra + 4096), P.f1 + j0, 2u * rb, bar);      // t_first
                lean_bulk(lean_s2u(s_extra + 8192), P.f2 + j0, 2u * rb, bar);      // aa
                lean_bulk(lean_s2u(s_extra + 12288), P.f3 + j0, 2u * rb, bar);     // bb
                lean_bulk(lean_s2u(s_extra + 16384), P.f4 + j0, 2u * rb, bar);     // pp
            }
        }
        if (cbytes) {
            lean_bulk(lean_s2u(s_rx), static_cast<const F*>(P.rx) + col0 + kc0, cbytes, bar);
            lean_bulk(lean_s2u(s_mx), static_cast<const F*>(P.mx) + col0 + kc0, cbytes, bar);
        }
    }
    MM8_STAMP(b.trace_id, blockIdx.x, 9);
    const uint8_t* wp = P.w + (long long)(j0 + sub) * P.w_stride + col0 + ch * 16;
    const long long step = (long long)rpp * P.w_stride;
    const uint32_t slot0 = lean_s2u(ring) + tid * 16;
#pragma unroll
    for (int g = 0; g < kDepthC; ++g) {
        if (active) {
#pragma unroll
            for (int u = 0; u < kGroup; ++u) {
                const int i = g * kGroup + u;
                if (sub + i * rpp < nrows) cp_async16(slot0 + i * (kThreads * 16), wp + i * step);
            }
        }
        cp_async_commit();
    }
    // rows past the end of the CTA's slice multiply with 0: clear the pairs (the barriers of the prologue
    // order this against the 16-bit stores below); the last columns of an odd-sized matrix come by plain loads
#pragma unroll
    for (int e = tid; e < ROWS; e += kThreads) xs[e] = 0;
    if (tid < kc1 - kc0 - ncol8) {
        s_rx[ncol8 + tid] = static_cast<const F*>(P.rx)[col0 + kc0 + ncol8 + tid];
        s_mx[ncol8 + tid] = static_cast<const F*>(P.mx)[col0 + kc0 + ncol8 + tid];
    }
    MM8_STAMP(b.trace_id, blockIdx.x, 0);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    MM8_STAMP(b.trace_id, blockIdx.x, 2);

    // ---- prologue ---------------------------------------------------------------------------------
    // what the epilogue adds or multiplies, for the (at most two) columns this thread finishes: on its way now
    float auxr[2] = {0.f, 0.f}, aux2r[2] = {0.f, 0.f};
    if (P.epilogue == RWKV_EPI_RESIDUAL || P.epilogue == RWKV_EPI_MUL_RESIDUAL) {
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int kk = kc0 + tid + it * kThreads;
            if (kk < kc1) {
                auxr[it] = ldc<F>(P.aux, col0 + kk);
                if (P.epilogue == RWKV_EPI_MUL_RESIDUAL) aux2r[it] = ldc<F>(P.aux2, col0 + kk);
            }
        }
    }
    const bool writer = panel == 0;
    float sx = 0.f, sxr = 0.f, sxmy = 0.f, xmax = 0.f;
    // Rows are dealt in pairs: thread t owns rows 2t, 2t + 1 (+ 512 per further round) of the CTA's slice, so that
    // every operand of a pair is one 32-bit (fp16 pair) or 64-bit (fp32 pair) access.
    constexpr int RPT = ROWS / kThreads;                 // rows per thread: 8 or 10
    constexpr int NI_PLAIN = RPT / 2, NI_STAGED = kLeanExtraRows / (2 * kThreads);
    float keep[RPT];                                     // this thread's x' (rows 2 * (tid + 256 i) + {0, 1})
    const __half2* ry2 = reinterpret_cast<const __half2*>(s_ry);
    const __half2* my2 = reinterpret_cast<const __half2*>(s_my);
    auto tail = [&](int slot, int lp, float2 xv) {       // x' = x * ry and the three sums the affine part needs
        const float2 ryf = __half22float2(ry2[lp]), myf = __half22float2(my2[lp]);
        const float xa = xv.x * ryf.x, xb = xv.y * ryf.y;
        keep[slot] = xa;
        keep[slot + 1] = xb;
        sx += xv.x + xv.y;
        sxr += xa + xb;
        sxmy = fmaf(xv.x, myf.x, fmaf(xv.y, myf.y, sxmy));
        xmax = fmaxf(xmax, fmaxf(fabsf(xa), fabsf(xb)));
    };
    auto wait_staged = [&]() {
        const uint32_t bar = lean_s2u(&mbar);
        unsigned it = 0;
        while (!lean_mbar_try(bar, 0)) {
            if (++it > (1u << 22)) { if (b.error) atomicExch(b.error, 1u); break; }
        }
    };
    if (P.prologue == RWKV_PRO_LN_MIX) {
        const __half* x = static_cast<const __half*>(P.x);
        F* s_xrow = reinterpret_cast<F*>(s_extra + 8192);
        const float shift = __half2float(__ldcg(x));     // statistics around x[0]: one pass without cancellation
        uint4 xv4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j8 = (tid + i * kThreads) * 8;     // the host guarantees N % 8 == 0 and N <= 8192
            xv4[i] = j8 < P.N ? __ldcg(reinterpret_cast<const uint4*>(x) + (j8 >> 3)) : make_uint4(0, 0, 0, 0);
        }
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j8 = (tid + i * kThreads) * 8;
            if (j8 < P.N) {
                const __half2* h = reinterpret_cast<const __half2*>(&xv4[i]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h[e]);
                    const float a = f.x - shift, c = f.y - shift;
                    s1 += a + c;
                    s2 = fmaf(a, a, s2);
                    s2 = fmaf(c, c, s2);
                }
                if (j8 >= j0 && j8 < j1) *reinterpret_cast<uint4*>(s_xrow + (j8 - j0)) = xv4[i];     // this CTA's rows
            }
        }
        s1 = warp_sum(s1); s2 = warp_sum(s2);
        if (lane == 0) { sh8[warp] = s1; sh8[kWarps + warp] = s2; }
        __syncthreads();
        wait_staged();
        MM8_STAMP(b.trace_id, blockIdx.x, 11);
        float t1 = 0.f, t2 = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < kWarps; ++w8) { t1 += sh8[w8]; t2 += sh8[kWarps + w8]; }
        const float dm = t1 * invn;
        const float mean = shift + dm;
        const float rstd = rsqrtf(fmaxf(fmaf(-dm, dm, t2 * invn), 0.f) + 1e-5f);
        const __half2* x2 = reinterpret_cast<const __half2*>(s_xrow);
        const __half2* lw2 = reinterpret_cast<const __half2*>(s_extra);
        const __half2* lb2 = reinterpret_cast<const __half2*>(s_extra + 2048);
        const __half2* mix2 = reinterpret_cast<const __half2*>(s_extra + 4096);
        const __half2* sx2 = reinterpret_cast<const __half2*>(s_extra + 6144);
        const int pmode = P.mode;
        const bool put_xx = writer && P.q0 != nullptr;
#pragma unroll
        for (int i = 0; i < NI_STAGED; ++i) {
            const int lp = tid + i * kThreads;
            if (2 * lp < nrows) {
                const float2 xf = __half22float2(x2[lp]), wf = __half22float2(lw2[lp]), bf = __half22float2(lb2[lp]);
                float2 xx;
                xx.x = r16((xf.x - mean) * rstd * wf.x + bf.x);
                xx.y = r16((xf.y - mean) * rstd * wf.y + bf.y);
                if (put_xx) reinterpret_cast<__half2*>(static_cast<__half*>(P.q0) + j0)[lp] = __floats2half2_rn(xx.x, xx.y);
                float2 xv = xx;
                if (pmode != 2) {
                    const float2 sv = __half22float2(sx2[lp]), mv = __half22float2(mix2[lp]);
                    if (pmode == 0) {
                        xv.x = r16(r16(xx.x * mv.x) + r16(sv.x * r16(1.0f - mv.x)));
                        xv.y = r16(r16(xx.y * mv.y) + r16(sv.y * r16(1.0f - mv.y)));
                    } else {
                        xv.x = r16(xx.x + r16(r16(sv.x - xx.x) * mv.x));
                        xv.y = r16(xx.y + r16(r16(sv.y - xx.y) * mv.y));
                    }
                }
                tail(2 * i, lp, xv);
            }
        }
    } else if (P.prologue == RWKV_PRO_WKV4) {            // pkg/model.py:1041-1055
        __half2 rr[NI_STAGED], kq[NI_STAGED], vq[NI_STAGED];
#pragma unroll
        for (int i = 0; i < NI_STAGED; ++i) {
            const int lp = tid + i * kThreads;
            if (2 * lp < nrows) {
                rr[i] = __ldcg(reinterpret_cast<const __half2*>(static_cast<const __half*>(P.x) + j0) + lp);
                kq[i] = __ldcg(reinterpret_cast<const __half2*>(static_cast<const __half*>(P.p0) + j0) + lp);
                vq[i] = __ldcg(reinterpret_cast<const __half2*>(static_cast<const __half*>(P.p1) + j0) + lp);
            }
        }
        wait_staged();
        const float2* td2 = reinterpret_cast<const float2*>(s_extra);
        const float2* tf2 = reinterpret_cast<const float2*>(s_extra + 4096);
        const float2* a2 = reinterpret_cast<const float2*>(s_extra + 8192);
        const float2* b2 = reinterpret_cast<const float2*>(s_extra + 12288);
        const float2* p2 = reinterpret_cast<const float2*>(s_extra + 16384);
        auto one = [&](float r, float kk, float vv, float a, float bq, float p0, float td, float tf, float& na, float& nb, float& np) {
            float ww = tf + kk;
            float p = fmaxf(p0, ww);
            float e1 = expf(p0 - p), e2 = expf(ww - p);
            const float wkv = r16((e1 * a + e2 * vv) / (e1 * bq + e2));
            if (writer) {                                // the new state: once per launch, by the CTAs of the first panel
                ww = td + p0;
                p = fmaxf(ww, kk);
                e1 = expf(ww - p); e2 = expf(kk - p);
                na = e1 * a + e2 * vv;
                nb = e1 * bq + e2;
                np = p;
            }
            return r16(r * wkv);
        };
#pragma unroll
        for (int i = 0; i < NI_STAGED; ++i) {
            const int lp = tid + i * kThreads;
            if (2 * lp < nrows) {
                const float2 r = __half22float2(rr[i]), kk = __half22float2(kq[i]), vv = __half22float2(vq[i]);
                const float2 a = a2[lp], bq = b2[lp], p0 = p2[lp], td = td2[lp], tf = tf2[lp];
                float2 na = make_float2(0.f, 0.f), nb = na, np = na, xv;
                xv.x = one(r.x, kk.x, vv.x, a.x, bq.x, p0.x, td.x, tf.x, na.x, nb.x, np.x);
                xv.y = one(r.y, kk.y, vv.y, a.y, bq.y, p0.y, td.y, tf.y, na.y, nb.y, np.y);
                if (writer) {
                    reinterpret_cast<float2*>(P.g0 + j0)[lp] = na;
                    reinterpret_cast<float2*>(P.g1 + j0)[lp] = nb;
                    reinterpret_cast<float2*>(P.g2 + j0)[lp] = np;
                }
                tail(2 * i, lp, xv);
            }
        }
    } else {
        __half2 xr[NI_PLAIN];
#pragma unroll
        for (int i = 0; i < NI_PLAIN; ++i) {
            const int lp = tid + i * kThreads;
            if (2 * lp < nrows) xr[i] = __ldcg(reinterpret_cast<const __half2*>(static_cast<const __half*>(P.x) + j0) + lp);
        }
        wait_staged();
#pragma unroll
        for (int i = 0; i < NI_PLAIN; ++i) {
            const int lp = tid + i * kThreads;
            if (2 * lp < nrows) tail(2 * i, lp, __half22float2(xr[i]));
        }
    }
    sx = warp_sum(sx); sxr = warp_sum(sxr); sxmy = warp_sum(sxmy); xmax = warp_max(xmax);
    if (lane == 0) { ssum[warp][0] = sx; ssum[warp][1] = sxr; ssum[warp][2] = sxmy; ssum[warp][3] = xmax; }
    __syncthreads();
    MM8_STAMP(b.trace_id, blockIdx.x, 3);
    // the staged vectors are not read again: the other ranks may overwrite them with their column sums
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    // x' as 16-bit fixed point: entry p * rpp + s of xs holds rows s + 2p * rpp (low half) and s + (2p + 1) * rpp
    // (high half), the two rows that the thread with row offset s multiplies in its p-th pair.  The range is the
    // largest that keeps a thread's 32-bit sums of `nsteps` products q * 255 from overflowing (32767 up to 257 steps).
    float xm = 0.f, xt = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < kWarps; ++w8) { xm = fmaxf(xm, ssum[w8][3]); xt += ssum[w8][1]; }
    if (!(xt == xt)) xm = __int_as_float(0x7f800000);    // a NaN does not show in a max but does in the sum
    const bool finite = xm < 3.0e38f;                    // false for inf and NaN
    const float scale = (finite && xm > 0.f) ? float(qmax) / xm : 0.f;
    const float inv_scale = !finite ? __int_as_float(0x7fc00000) : xm > 0.f ? xm / float(qmax) : 0.f;
    {
        uint16_t* xq16 = reinterpret_cast<uint16_t*>(xs);
        const int ni = (P.prologue == RWKV_PRO_PLAIN) ? NI_PLAIN : NI_STAGED;
#pragma unroll
        for (int i = 0; i < NI_PLAIN; ++i) {
            const int l = 2 * (tid + i * kThreads);
            if (i < ni && l < nrows) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int st = fast_div(l + e, rpp, m_rpp), so = l + e - st * rpp;
                    xq16[(((st >> 1) * rpp + so) << 1) + (st & 1)] = uint16_t(__float2int_rn(keep[2 * i + e] * scale));
                }
            }
        }
    }
    __syncthreads();
    MM8_STAMP(b.trace_id, blockIdx.x, 13);

    // ---- main loop: two rows per step, exact integer sums (mm8_core.cuh) -----------------------------
    float acc[16];
    {
        int iacc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) iacc[i] = 0;
        int sq = 0;
        const int* xq_ptr = xs + sub;
        const uint8_t* wn = wp + (long long)(kDepthC * kGroup) * step;
        const long long step2 = 2 * step, step3 = 3 * step;
        int inext = kDepthC * kGroup;
        uint32_t rd = 0;
        for (int g = 0; g < ngroups; ++g) {
            cp_async_wait<kDepthC - 1>();
            const uint8_t* rb = ring + tid * 16 + rd;
            uint4 v[kGroup];
#pragma unroll
            for (int u = 0; u < kGroup; ++u) v[u] = *reinterpret_cast<const uint4*>(rb + u * (kThreads * 16));
            if (active) {
                const int xq0 = xq_ptr[0], xq1 = xq_ptr[rpp];                   // 0 for rows past the end
                xq_ptr += 2 * rpp;
                dot16_q(iacc, v[0], v[1], xq0);
                dot16_q(iacc, v[2], v[3], xq1);
                sq = dp2a_lo(xq0, 0x00000101u, sq);
                sq = dp2a_lo(xq1, 0x00000101u, sq);
            }
            {   // refill the position just drained with group g + kDepthC
                const uint32_t dst = slot0 + rd;
                if (inext < cnt) cp_async16(dst, wn);
                if (inext + 1 < cnt) cp_async16(dst + kThreads * 16, wn + step);
                if (inext + 2 < cnt) cp_async16(dst + 2 * kThreads * 16, wn + step2);
                if (inext + 3 < cnt) cp_async16(dst + 3 * kThreads * 16, wn + step3);
                cp_async_commit();
                wn += 4 * step;
                inext += kGroup;
            }
            rd += kGroup * kThreads * 16;
            if (rd == uint32_t(kDepthC * kGroup * kThreads * 16)) rd = 0;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = float(iacc[i] - 128 * sq) * inv_scale;
    }
    cp_async_wait<0>();
    MM8_STAMP(b.trace_id, blockIdx.x, 4);

    // ---- CTA reduce: thread t leaves its 16 sums at red[t * 20] (the stride keeps the 16-byte stores
    // of a warp on distinct banks); column c * 16 + i of row group rg is red[(rg * cpr + c) * 20 + i].
    __syncthreads();                                     // every thread is done with its ring
    float* red = reinterpret_cast<float*>(ring);         // [rpp][cpr][20]   <= 20 KB
    if (active) {
        float4* dst = reinterpret_cast<float4*>(red + tid * 20);
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[q] = make_float4(acc[q * 4], acc[q * 4 + 1], acc[q * 4 + 2], acc[q * 4 + 3]);
    }
    __syncthreads();
    MM8_STAMP(b.trace_id, blockIdx.x, 12);
    // every CTA of the cluster is past its prologue: its stage area may now receive column sums
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    MM8_STAMP(b.trace_id, blockIdx.x, 8);
    {
        const uint32_t gat = lean_s2u(gather) + uint32_t(rank * per) * 4u;
        for (int kk = tid; kk < ncols; kk += kThreads) {
            const float* src = red + (kk >> 4) * 20 + (kk & 15);
            float s = 0.f;
#pragma unroll 4
            for (int rg = 0; rg < rpp; ++rg) s += src[rg * cpr * 20];
            const int q = int(__umulhi(unsigned(kk), m_per));           // the rank that finishes column kk
            st_remote_f32(gat + uint32_t(kk - q * per) * 4u, uint32_t(q), s);
        }
        if (tid < 4 * S && (tid & 3) < 3) {
            float s = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < kWarps; ++w8) s += ssum[w8][tid & 3];
            st_remote_f32(lean_s2u(&gat3[rank][tid & 3]), uint32_t(tid >> 2), s);
        }
    }
    MM8_STAMP(b.trace_id, blockIdx.x, 14);
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    MM8_STAMP(b.trace_id, blockIdx.x, 5);

    // ---- finish this CTA's columns: the ranks' sums in rank order (bit-reproducible), affine tail, epilogue
    float tx = 0.f, txr = 0.f, txmy = 0.f;
    if (S == kMaxClusterSize) {                          // the usual case, unrolled: all loads first
#pragma unroll
        for (int q = 0; q < kMaxClusterSize; ++q) { tx += gat3[q][0]; txr += gat3[q][1]; txmy += gat3[q][2]; }
    } else {
        for (int q = 0; q < S; ++q) { tx += gat3[q][0]; txr += gat3[q][1]; txmy += gat3[q][2]; }
    }
#pragma unroll
    for (int it = 0; it < 2; ++it) {
        const int kk = kc0 + tid + it * kThreads;
        if (kk < kc1) {
            const int e = kk - kc0;
            float s = 0.f;
            if (S == kMaxClusterSize) {
#pragma unroll
                for (int q = 0; q < kMaxClusterSize; ++q) s += gather[q * per + e];
            } else {
                for (int q = 0; q < S; ++q) s += gather[q * per + e];
            }
            const float rxk = __half2float(s_rx[e]), mxk = __half2float(s_mx[e]);
            const float val = fmaf(rxk, s, fmaf(rxk * 128.5f, txr, fmaf(mxk, tx, txmy)));
            store_epilogue_with<F>(P, col0 + kk, val, auxr[it], aux2r[it]);
        }
    }
    MM8_STAMP(b.trace_id, blockIdx.x, 6);
    MM8_STAMP(b.trace_id, blockIdx.x, 7);
}

// The device's error word (NULL if it cannot be resolved); resolved once per device.
static inline unsigned* lean_error_word() {
    static unsigned* word[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return nullptr; }
    if (word[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_lean_error) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        word[dev] = static_cast<unsigned*>(p);
    }
    return word[dev];
}

// Launch on the lean kernel if every problem qualifies; RWKV_ERR_UNSUPPORTED sends the caller to mm8_cluster_kernel.
static inline bool lean_aligned16(const void* p) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static inline int mm8_lean_launch(const Batch& plan_b, int count, bool wide_hint, cudaStream_t st) {
    if (g_use_lean < 0) {
        const char* e = getenv("RWKV_B200_LEAN");
        g_use_lean = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    if (!g_use_lean || g_cluster_size < 0) return RWKV_ERR_UNSUPPORTED;
    LeanBatch lb;
    memset(&lb, 0, sizeof(lb));
    int min_n = INT32_MAX, max_n = 0;
    long long total_cols = 0;
    for (int i = 0; i < count; ++i) {
        const Problem& q = plan_b.p[i];
        lb.p[i] = q;
        if (q.N < min_n) min_n = q.N;
        if (q.N > max_n) max_n = q.N;
        total_cols += q.M;
        if (q.N % 8 != 0) return RWKV_ERR_UNSUPPORTED;
        if (!lean_aligned16(q.ry) || !lean_aligned16(q.my) || !lean_aligned16(q.rx) || !lean_aligned16(q.mx)) return RWKV_ERR_UNSUPPORTED;
        if (q.prologue == RWKV_PRO_LN_MIX) {
            if (!lean_aligned16(q.p0) || !lean_aligned16(q.p1) || !lean_aligned16(q.x)) return RWKV_ERR_UNSUPPORTED;
            if (q.mode != 2 && (!lean_aligned16(q.p2) || !lean_aligned16(q.p3))) return RWKV_ERR_UNSUPPORTED;
            if (q.q0 != nullptr && (reinterpret_cast<uintptr_t>(q.q0) & 3) != 0) return RWKV_ERR_UNSUPPORTED;
        } else if (q.prologue == RWKV_PRO_WKV4) {
            if (!lean_aligned16(q.f0) || !lean_aligned16(q.f1) || !lean_aligned16(q.f2) || !lean_aligned16(q.f3) || !lean_aligned16(q.f4))
                return RWKV_ERR_UNSUPPORTED;
            // rows go in pairs: fp16 pairs of r, k, v and fp32 pairs of the new state
            if (((reinterpret_cast<uintptr_t>(q.x) | reinterpret_cast<uintptr_t>(q.p0) | reinterpret_cast<uintptr_t>(q.p1)) & 3) != 0 ||
                ((reinterpret_cast<uintptr_t>(q.g0) | reinterpret_cast<uintptr_t>(q.g1) | reinterpret_cast<uintptr_t>(q.g2)) & 7) != 0)
                return RWKV_ERR_UNSUPPORTED;
        } else if ((reinterpret_cast<uintptr_t>(q.x) & 3) != 0) {
            return RWKV_ERR_UNSUPPORTED;
        }
    }
    for (int i = count; i < kMaxProblems; ++i) lb.p[i] = lb.p[0];
    int S = g_cluster_size > 0 ? g_cluster_size : kMaxClusterSize;
    if (S != 1 && S != 2 && S != 4 && S != 8) return RWKV_ERR_UNSUPPORTED;
    if (g_cluster_size == 0) while (S > 1 && min_n < S * 64) S >>= 1;
    const int rows_needed = ((max_n + S - 1) / S + 7) & ~7;
    if (rows_needed > kWideRowsPerCta) return RWKV_ERR_UNSUPPORTED;
    const bool wide = rows_needed > kMaxRowsPerCta || wide_hint;
    for (int i = 0; i < count; ++i) {
        const int rows = ((lb.p[i].N + S - 1) / S + 7) & ~7;
        if (lb.p[i].prologue != RWKV_PRO_PLAIN && rows > kLeanExtraRows) return RWKV_ERR_UNSUPPORTED;
    }
    void (*kern)(LeanBatch) = wide ? mm8_lean_kernel<kWideRowsPerCta> : mm8_lean_kernel<kMaxRowsPerCta>;
    const int smem = wide ? cluster_smem<kWideRowsPerCta>() : cluster_smem<kMaxRowsPerCta>();
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
        cudaGetLastError();
        return RWKV_ERR_UNSUPPORTED;
    }
    int slots = cluster_slots(kern, S, smem, wide);
    if (slots <= 0) return RWKV_ERR_UNSUPPORTED;
    // Planning as in mm8_cluster_launch: launches of several matrices take four fifths of the resident clusters
    // (the free slots let the successor's first clusters fill their rings early); a launch of ONE matrix takes
    // all of them (measured at the 7B shape: 608 -> 618 tok/s; with every launch on all slots: 600).
    {
        int planned = 0;
        for (int i = 0; i < g_plan_n; ++i) if (g_plan[i].cols == total_cols) planned = g_plan[i].clusters;
        if (planned > 0) { if (planned < slots) slots = planned; }
        else if (g_cluster_pw < 0) { if (-g_cluster_pw < slots) slots = -g_cluster_pw; }
        else if (g_cluster_pw == 0 && slots >= 10 && count > 1) slots = slots * 4 / 5;
    }
    int pw = g_cluster_pw > 0 ? (g_cluster_pw + 15) / 16 * 16 : 16;
    if (pw > kMaxPanelCols) pw = kMaxPanelCols;
    if (g_cluster_pw <= 0) {
        long long guess = (total_cols + slots - 1) / slots;
        pw = int((guess + 15) / 16 * 16);
        if (pw < 16) pw = 16;
        for (; pw < kMaxPanelCols; pw += 16) {
            int panels = 0;
            for (int i = 0; i < count; ++i) panels += (lb.p[i].M + pw - 1) / pw;
            if (panels <= slots) break;
        }
        if (pw > kMaxPanelCols) pw = kMaxPanelCols;
    }
    if (((((pw + S - 1) / S) + 7) & ~7) > kStageEpiCols) return RWKV_ERR_UNSUPPORTED;
    lb.pw = pw;
    lb.S = S;
    lb.s_log2 = S == 8 ? 3 : S == 4 ? 2 : S == 2 ? 1 : 0;
    lb.cpr = pw / 16;
    lb.rpp = kThreads / lb.cpr;
    lb.m_cpr = 0xffffffffu / unsigned(lb.cpr) + 1u;
    lb.m_rpp = 0xffffffffu / unsigned(lb.rpp) + 1u;
    lb.panel_start[0] = 0;
    for (int i = 0; i < kMaxProblems; ++i) {
        const int panels = i < count ? (lb.p[i].M + pw - 1) / pw : 0;
        lb.panel_start[i + 1] = lb.panel_start[i] + panels;
        if (i < count) {
            lb.p[i].rows_per_cta = ((lb.p[i].N + S - 1) / S + 7) & ~7;
            lb.p[i].splits = S;
        }
    }
    const long long ctas = (long long)lb.panel_start[kMaxProblems] * S;
    if (ctas > INT32_MAX) return RWKV_ERR_UNSUPPORTED;
    lb.error = lean_error_word();

    static int use_pdl = -1;
    if (use_pdl < 0) {
        const char* e = getenv("RWKV_B200_PDL");
        use_pdl = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(ctas));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = size_t(smem);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = unsigned(S);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 2 : 1;
    lb.trace_id = 0;
#ifdef RWKV_MM8_TRACE
    lb.trace_id = g_mm8_trace_next++;
#endif
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, lb);
    if (e != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    return RWKV_OK;
}

}  // namespace
