// mm8_one with the K-split reduced inside a thread-block cluster.
//
// Same algebra, ring, prologues and epilogues as mm8_one_kernel (mm8_one.cu); what differs is
// how the K-splits of a column panel meet.  There the splits of a panel are unrelated CTAs that
// exchange partial sums through global scratch and an atomic ticket: three dependent trips to L2
// on the critical path of every launch, each ~3 us when the HBM is saturated.  Here the S <= 8
// splits of a panel ARE one cluster: after the stream every CTA leaves its column sums in its
// own shared memory, one cluster barrier later each CTA adds the S copies of ITS 1/S of the
// panel's columns through distributed shared memory (in rank order: bit-reproducible) and
// applies the epilogue.  No scratch, no ticket, no global round trip.
//
// Panels: the width is any multiple of 16 columns, chosen by the host so that one wave of
// clusters covers all matrices of the launch (e.g. 37 clusters x 8 CTAs on 148 SMs x 2).  A row
// of a panel is `cpr` 16-byte chunks; thread t owns chunk t % cpr of rows t / cpr, t / cpr + rpp,
// ... (rpp = 256 / cpr rows per CTA step), so any width keeps nearly all threads busy.
#pragma once
#include <cooperative_groups.h>
#include <string.h>

#include "mm8_core.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int kDepthC = 4;
constexpr int kMaxPanelCols = 4096;          // cpr <= 256
constexpr int kMaxClusterSize = 8;

struct ClusterBatch {
    Problem p[kMaxProblems];
    int panel_start[kMaxProblems + 1];       // cumulative panel counts
    int pw;                                  // panel width in columns (multiple of 16)
    int S;                                   // cluster size = K-splits
    int trace_id;
};

// Shared-memory plan behind the 64 KB ring (bytes; F = activation type):
//   [0, 2R*sF)            ry, my of this CTA's rows (R = 2048 rows at most)
//   [2R*sF, +8 KB)        LN_MIX: ln weight, ln bias, mix (fp16);  WKV4: t_decay, t_first (fp32)
//                         -- only when the CTA has at most 1024 rows, else read from global memory
//   [.., +4*512*sF)       rx, mx, aux, aux2 of the columns this CTA finishes (at most 512)
// Everything that is a model constant is copied here BEFORE the wait on the preceding kernel.
constexpr int kStageExtraRows = 1024;
constexpr int kStageExtraBytes = 8192;
constexpr int kStageEpiCols = 512;
template <typename F, int ROWS> constexpr int stage_bytes() { return 2 * ROWS * int(sizeof(F)) + kStageExtraBytes + 4 * kStageEpiCols * int(sizeof(F)); }
// dynamic shared memory: what caps residency at two CTAs per SM, less when x' needs more static room
template <int ROWS> constexpr int cluster_smem() { return ROWS <= kMaxRowsPerCta ? 104 * 1024 : 102 * 1024; }

// Multi-GPU form (one model split by output columns over the ranks, one process per GPU): the
// epilogue stores every result into the same place of every other rank's activation buffer as
// well (plain stores to peer memory over NVLink), the last CTA of the launch to finish then writes
// the launch's sequence number into each rank's arrival word for this rank, and the prologue of
// the NEXT launch waits (bounded) until every rank's word has reached the number it needs.  The
// all-gather that a column-sharded matmul needs thus happens inside the matmul kernels: no
// collective call, no extra launch, transfers overlap the tail of the stream tile by tile.
struct Exchange {
    void* peer_y[kMaxProblems][7];
    unsigned* arrived;           // this rank's arrival words [world]
    unsigned* peer_arrived[7];   // on each other rank: its arrival word for this rank
    unsigned* done_counter;
    unsigned* error;
    const unsigned* seq_base;    // added to wait_seq / signal_seq (device word; lets a captured graph be replayed)
    unsigned wait_seq, signal_seq;
    int world, rank, n_peers;
};
struct NoExchange { int unused; };
constexpr unsigned kPeerSpinLimit = 1u << 21;

// MODE: 0 = scalar fp32, 1 = two-wide fp32 instructions, 2 = 16-bit fixed-point activations and dp2a
template <typename F, int MODE, typename EX, int ROWS>
__global__ void __launch_bounds__(kThreads, 2) mm8_cluster_kernel(const __grid_constant__ ClusterBatch b, const __grid_constant__ EX ex) {
    constexpr bool kExch = sizeof(EX) > sizeof(NoExchange);
    asm volatile("griddepcontrol.launch_dependents;");
    MM8_TRACE_BEGIN(b.trace_id, blockIdx.x);
    cg::cluster_group cluster = cg::this_cluster();
    const int S = b.S;
    const int rank = int(cluster.block_rank());
    const int cid = int(blockIdx.x) / S;
    int z = 0;
    while (z + 1 < kMaxProblems && cid >= b.panel_start[z + 1]) ++z;
    const Problem& P = b.p[z];
    const int panel = cid - b.panel_start[z];
    const int col0 = panel * b.pw;
    const int ncols = min(b.pw, P.M - col0);             // >= 1 by construction of the grid
    const int cpr = (ncols + 15) >> 4;                   // 16-byte chunks per panel row
    const int rpp = kThreads / cpr;                      // rows per CTA step
    const int PWc = cpr * 16;

    extern __shared__ __align__(128) uint8_t ring[];    // [slot][thread] 16 B; later the reduce buffers
    static_assert(ring_bytes(kDepthC) + stage_bytes<F, ROWS>() <= cluster_smem<ROWS>(), "stage area does not fit");
    __shared__ float xs[ROWS];
    __shared__ float ssum[kWarps][3];
    __shared__ float sh8[kWarps];
    __shared__ float smax[kWarps];                       // per warp: largest |x'|
    __shared__ float tot3[4];                            // this CTA's scalar sums (read by the cluster)
    __shared__ float all3[4];                            // the cluster's scalar sums

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j0 = rank * P.rows_per_cta;                // rows_per_cta is a multiple of 8
    const int j1 = min(P.N, j0 + P.rows_per_cta);
    const int nrows = max(0, j1 - j0);
    const int sub = tid / cpr;                           // this thread's row within a CTA step
    const int ch = tid - sub * cpr;                      // this thread's chunk within the row
    const bool active = sub < rpp;
    const int nsteps = (nrows + rpp - 1) / rpp;
    const int ngroups = (nsteps + kGroup - 1) / kGroup;
    const uint8_t* wp = P.w + (long long)(j0 + sub) * P.w_stride + col0 + ch * 16;
    const long long step = (long long)rpp * P.w_stride;
    const uint32_t slot0 = (uint32_t)__cvta_generic_to_shared(ring) + tid * 16;

    // columns this CTA finishes after the cluster reduction: [kc0, kc1) of the panel
    const int per = ((ncols + S - 1) / S + 7) & ~7;
    const int kc0 = min(ncols, rank * per), kc1 = min(ncols, kc0 + per);
    const bool epi_staged = per <= kStageEpiCols;
    const bool extra_staged = nrows <= kStageExtraRows;

    uint8_t* stage = ring + ring_bytes(kDepthC);
    F* s_ry = reinterpret_cast<F*>(stage);
    F* s_my = s_ry + ROWS;
    uint8_t* s_extra = stage + 2 * ROWS * sizeof(F);
    F* s_rx = reinterpret_cast<F*>(s_extra + kStageExtraBytes);
    F* s_mx = s_rx + kStageEpiCols;
    F* s_aux = s_mx + kStageEpiCols;
    F* s_aux2 = s_aux + kStageEpiCols;

    // ---- before the preceding kernel is known to be done: model constants only -------------
    stage_vec<sizeof(F)>(reinterpret_cast<uint8_t*>(s_ry), P.ry, j0, nrows, tid);
    stage_vec<sizeof(F)>(reinterpret_cast<uint8_t*>(s_my), P.my, j0, nrows, tid);
    if (extra_staged) {
        if (P.prologue == RWKV_PRO_LN_MIX) {
            stage_vec<2>(s_extra, P.p0, j0, nrows, tid);                                   // ln weight
            stage_vec<2>(s_extra + 2 * kStageExtraRows, P.p1, j0, nrows, tid);             // ln bias
            if (P.mode != 2) stage_vec<2>(s_extra + 4 * kStageExtraRows, P.p3, j0, nrows, tid);   // mix
        } else if (P.prologue == RWKV_PRO_WKV4) {
            stage_vec<4>(s_extra, P.f0, j0, nrows, tid);                                   // t_decay
            stage_vec<4>(s_extra + 4 * kStageExtraRows, P.f1, j0, nrows, tid);             // t_first
        }
    }
    if (epi_staged) {
        stage_vec<sizeof(F)>(reinterpret_cast<uint8_t*>(s_rx), P.rx, col0 + kc0, kc1 - kc0, tid);
        stage_vec<sizeof(F)>(reinterpret_cast<uint8_t*>(s_mx), P.mx, col0 + kc0, kc1 - kc0, tid);
    }
    cp_async_commit();

    auto issue_group = [&](int g) {
        if (active) {
#pragma unroll
            for (int u = 0; u < kGroup; ++u) {
                const int i = g * kGroup + u;
                if (sub + i * rpp < nrows) cp_async16(slot0 + ((g % kDepthC) * kGroup + u) * (kThreads * 16), wp + i * step);
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int g = 0; g < kDepthC; ++g) issue_group(g);
    // State of the previous token (token-shift vector, WKV accumulators) is usually in DRAM by now:
    // pull its lines into L2.  A hint only; the loads themselves come after the wait.
    if (P.prologue == RWKV_PRO_LN_MIX && P.mode != 2) l2_prefetch<2>(P.p2, j0, nrows, tid);
    if (P.prologue == RWKV_PRO_WKV4) {
        l2_prefetch<4>(P.f2, j0, nrows, tid);
        l2_prefetch<4>(P.f3, j0, nrows, tid);
        l2_prefetch<4>(P.f4, j0, nrows, tid);
    }
    MM8_STAMP(b.trace_id, blockIdx.x, 0);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    MM8_STAMP(b.trace_id, blockIdx.x, 2);
    if constexpr (kExch) {
        // the other ranks' slices of this launch's inputs: wait for their arrival words (bounded)
        if (ex.wait_seq != 0 && tid < ex.world) {
            const unsigned want = ex.wait_seq + (ex.seq_base ? __ldcg(ex.seq_base) : 0u);
            unsigned it = 0;
            while (true) {
                unsigned v;
                asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ex.arrived + tid) : "memory");
                if (int(v - want) >= 0) break;
                if (++it >= kPeerSpinLimit) { atomicExch(ex.error, 1u); break; }
                __nanosleep(32);
            }
            __threadfence_system();              // acquire: what the ranks stored before their words is visible
        }
        __syncthreads();
    }

    // ---- prologue: one trip to L2 for what earlier kernels wrote, then x' = x * ry ----------
    const bool writer = panel == 0;
    float sx = 0.f, sxr = 0.f, sxmy = 0.f, xmax = 0.f;      // xmax: largest |x'| (NaN-propagating max is not needed: see quantize_pairs)
    if (P.prologue == RWKV_PRO_LN_MIX) {
        const __half* x = static_cast<const __half*>(P.x);
        const int nvec = P.N / 8;               // host guarantees N % 8 == 0 and N <= 8192
        uint4 xv4[4], sv4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j8 = (tid + i * kThreads) * 8;
            xv4[i] = j8 < P.N ? __ldcg(reinterpret_cast<const uint4*>(x) + (j8 >> 3)) : make_uint4(0, 0, 0, 0);
            // previous token's vector for the rows of this CTA (j0 and nrows are multiples of 8
            // except for the tail of the last rank, which N % 8 == 0 keeps whole)
            sv4[i] = (P.mode != 2 && j8 >= j0 && j8 < j1) ? __ldcg(reinterpret_cast<const uint4*>(P.p2) + (j8 >> 3))
                                                          : make_uint4(0, 0, 0, 0);
        }
        (void)nvec;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2* h = reinterpret_cast<const __half2*>(&xv4[i]);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h[e]); s += f.x + f.y; }
        }
        cp_async_wait<kDepthC>();               // the staged constants have landed (block_sum256 publishes them)
        const float mean = block_sum256(s, sh8) / float(P.N);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if ((tid + i * kThreads) * 8 < P.N) {
                const __half2* h = reinterpret_cast<const __half2*>(&xv4[i]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h[e]);
                    q = fmaf(f.x - mean, f.x - mean, q);
                    q = fmaf(f.y - mean, f.y - mean, q);
                }
            }
        }
        const float rstd = rsqrtf(block_sum256(q, sh8) / float(P.N) + 1e-5f);
        const __half* lw = extra_staged ? reinterpret_cast<const __half*>(s_extra) : static_cast<const __half*>(P.p0) + j0;
        const __half* lb = extra_staged ? reinterpret_cast<const __half*>(s_extra + 2 * kStageExtraRows) : static_cast<const __half*>(P.p1) + j0;
        const __half* mixv = P.mode == 2 ? nullptr
                           : extra_staged ? reinterpret_cast<const __half*>(s_extra + 4 * kStageExtraRows) : static_cast<const __half*>(P.p3) + j0;
        // the rows of this CTA are computed by whichever thread holds them in registers
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j8 = (tid + i * kThreads) * 8;
            if (j8 >= j0 && j8 < j1) {
                const __half* hx = reinterpret_cast<const __half*>(&xv4[i]);
                const __half* hs = reinterpret_cast<const __half*>(&sv4[i]);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int l = j8 + e - j0;
                    const float xx = r16((__half2float(hx[e]) - mean) * rstd * __half2float(lw[l]) + __half2float(lb[l]));
                    if (writer && P.q0) static_cast<__half*>(P.q0)[j8 + e] = __float2half_rn(xx);
                    float xv = xx;
                    if (P.mode != 2) {
                        const float sxv = __half2float(hs[e]), mv = __half2float(mixv[l]);
                        xv = P.mode == 0 ? r16(r16(xx * mv) + r16(sxv * r16(1.0f - mv))) : r16(xx + r16(r16(sxv - xx) * mv));
                    }
                    const float xp = xv * to_f32<F>(s_ry[l]);
                    xs[l] = xp;
                    sx += xv;
                    sxr += xp;
                    sxmy = fmaf(xv, to_f32<F>(s_my[l]), sxmy);
                    xmax = fmaxf(xmax, fabsf(xp));
                }
            }
        }
    } else if (P.prologue == RWKV_PRO_WKV4) {        // pkg/model.py:1041-1055
        cp_async_wait<kDepthC>();               // the staged constants have landed
        __syncthreads();
        const float* tdv = extra_staged ? reinterpret_cast<const float*>(s_extra) : P.f0 + j0;
        const float* tfv = extra_staged ? reinterpret_cast<const float*>(s_extra + 4 * kStageExtraRows) : P.f1 + j0;
#pragma unroll 2
        for (int l = tid; l < nrows; l += kThreads) {
            const int j = j0 + l;
            const float r = ldc<__half>(P.x, j), kk = ldc<__half>(P.p0, j), vv = ldc<__half>(P.p1, j);
            const float a = __ldcg(P.f2 + j), bq = __ldcg(P.f3 + j), p0 = __ldcg(P.f4 + j);
            float ww = tfv[l] + kk;
            float p = fmaxf(p0, ww);
            float e1 = expf(p0 - p), e2 = expf(ww - p);
            const float wkv = r16((e1 * a + e2 * vv) / (e1 * bq + e2));
            if (writer) {
                ww = tdv[l] + p0;
                p = fmaxf(ww, kk);
                e1 = expf(ww - p); e2 = expf(kk - p);
                P.g0[j] = e1 * a + e2 * vv;
                P.g1[j] = e1 * bq + e2;
                P.g2[j] = p;
            }
            const float xv = r16(r * wkv);
            const float xp = xv * to_f32<F>(s_ry[l]);
            xs[l] = xp;
            sx += xv;
            sxr += xp;
            sxmy = fmaf(xv, to_f32<F>(s_my[l]), sxmy);
            xmax = fmaxf(xmax, fabsf(xp));
        }
    } else {
        // all loads of a thread first (independent: one trip), then the arithmetic
        constexpr int RPT = ROWS / kThreads;             // rows per thread: 8 or 10
        float xr[RPT];
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            const int l = tid + i * kThreads;
            xr[i] = l < nrows ? ldc<F>(P.x, j0 + l) : 0.f;
        }
        cp_async_wait<kDepthC>();               // the staged constants have landed
        __syncthreads();
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            const int l = tid + i * kThreads;
            if (l < nrows) {
                const float xv = xr[i];
                const float xp = xv * to_f32<F>(s_ry[l]);
                xs[l] = xp;
                sx += xv;
                sxr += xp;
                sxmy = fmaf(xv, to_f32<F>(s_my[l]), sxmy);
                xmax = fmaxf(xmax, fabsf(xp));
            }
        }
    }
    // what the epilogue adds or multiplies (written by earlier kernels): on its way during the stream
    if (epi_staged) {
        if (P.epilogue == RWKV_EPI_RESIDUAL || P.epilogue == RWKV_EPI_MUL_RESIDUAL)
            stage_vec<sizeof(F)>(reinterpret_cast<uint8_t*>(s_aux), P.aux, col0 + kc0, kc1 - kc0, tid);
        if (P.epilogue == RWKV_EPI_MUL_RESIDUAL)
            stage_vec<sizeof(F)>(reinterpret_cast<uint8_t*>(s_aux2), P.aux2, col0 + kc0, kc1 - kc0, tid);
    }
    cp_async_commit();
    sx = warp_sum(sx); sxr = warp_sum(sxr); sxmy = warp_sum(sxmy); xmax = warp_max(xmax);
    if (lane == 0) { ssum[warp][0] = sx; ssum[warp][1] = sxr; ssum[warp][2] = sxmy; smax[warp] = xmax; }
    __syncthreads();
    MM8_STAMP(b.trace_id, blockIdx.x, 3);

    // ---- main loop ---------------------------------------------------------------------------
    float acc[16];
    if (MODE == 2) {
        // integer form: x' as 16-bit fixed point, two rows per step (mm8_core.cuh)
        // largest |x'| of the CTA from the warps' maxima; a NaN does not show in a max but does in the sum
        float xm = 0.f, xt = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < kWarps; ++w8) { xm = fmaxf(xm, smax[w8]); xt += ssum[w8][1]; }
        if (!(xt == xt)) xm = __int_as_float(0x7f800000);
        const float inv_scale = quantize_pairs<ROWS <= 2048 ? 8 : 10>(xs, rpp, cpr, sub, ch, active, ngroups * (kGroup / 2), nsteps, nrows, xm);
        int iacc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) iacc[i] = 0;
        int sq = 0;
        // running state instead of per-iteration index arithmetic: the ring position being drained,
        // this thread's next pair of activations, and the rows of the group to fetch next
        const int cnt = (active && sub < nrows) ? (nrows - sub + rpp - 1) / rpp : 0;     // rows of this thread
        const int* xq_ptr = reinterpret_cast<const int*>(xs) + sub;
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
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
        for (int g = 0; g < ngroups; ++g) {
            cp_async_wait<kDepthC - 1>();
            uint4 v[kGroup];
#pragma unroll
            for (int u = 0; u < kGroup; ++u)
                v[u] = *reinterpret_cast<const uint4*>(ring + tid * 16 + ((g % kDepthC) * kGroup + u) * (kThreads * 16));
            if (active) {
#pragma unroll
                for (int u = 0; u < kGroup; ++u) {
                    const int r = sub + (g * kGroup + u) * rpp;
                    if (r < nrows) fma16<MODE == 1>(acc, v[u], xs[r]);
                }
            }
            issue_group(g + kDepthC);
        }
    }
    cp_async_wait<0>();
    MM8_STAMP(b.trace_id, blockIdx.x, 4);

    // ---- CTA reduce.  Row group rg keeps column c*16 + i of the panel at rg*PWc + c*16 +
    // ((i + c) & 15): the rotation spreads a warp's stores over the banks, and the column-order
    // reads below are conflict free.
    __syncthreads();                             // every thread is done with its ring
    float* red = reinterpret_cast<float*>(ring);                 // [rpp][PWc]   <= 16 KB
    float* cs = reinterpret_cast<float*>(ring + 16384);          // [PWc] column sums of this CTA
    if (active) {
#pragma unroll
        for (int i = 0; i < 16; ++i) red[sub * PWc + ch * 16 + ((i + ch) & 15)] = acc[i];
    }
    __syncthreads();
    for (int kk = tid; kk < PWc; kk += kThreads) {
        const int pos = (kk & ~15) + (((kk & 15) + (kk >> 4)) & 15);
        float s = 0.f;
        for (int rg = 0; rg < rpp; ++rg) s += red[rg * PWc + pos];
        cs[kk] = s;
    }
    if (tid < 3) {
        float s = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < kWarps; ++w8) s += ssum[w8][tid];
        tot3[tid] = s;
    }
    cluster.sync();                              // every CTA's cs / tot3 are complete and visible
    MM8_STAMP(b.trace_id, blockIdx.x, 5);

    // ---- cluster reduce through distributed shared memory, in rank order --------------------
    if (warp == 0) {
        float v0 = 0.f, v1 = 0.f, v2 = 0.f;
        if (lane < S) {
            const float* rt = cluster.map_shared_rank(tot3, lane);
            v0 = rt[0]; v1 = rt[1]; v2 = rt[2];
        }
        float t0 = 0.f, t1 = 0.f, t2 = 0.f;
        for (int q = 0; q < S; ++q) {
            t0 += __shfl_sync(0xffffffffu, v0, q);
            t1 += __shfl_sync(0xffffffffu, v1, q);
            t2 += __shfl_sync(0xffffffffu, v2, q);
        }
        if (lane == 0) { all3[0] = t0; all3[1] = t1; all3[2] = t2; }
    }
    __syncthreads();
    const float tx = all3[0], txr = all3[1], txmy = all3[2];
    for (int kk = kc0 + tid; kk < kc1; kk += kThreads) {
        float a[kMaxClusterSize];
#pragma unroll
        for (int q = 0; q < kMaxClusterSize; ++q) a[q] = q < S ? cluster.map_shared_rank(cs, q)[kk] : 0.f;
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < kMaxClusterSize; ++q) s += a[q];
        const int k = col0 + kk, e = kk - kc0;
        float rxk, mxk, auxv = 0.f, aux2v = 0.f;
        if (epi_staged) {
            rxk = to_f32<F>(s_rx[e]); mxk = to_f32<F>(s_mx[e]);
            if (P.epilogue == RWKV_EPI_RESIDUAL || P.epilogue == RWKV_EPI_MUL_RESIDUAL) auxv = to_f32<F>(s_aux[e]);
            if (P.epilogue == RWKV_EPI_MUL_RESIDUAL) aux2v = to_f32<F>(s_aux2[e]);
        } else {
            rxk = to_f32<F>(static_cast<const F*>(P.rx)[k]); mxk = to_f32<F>(static_cast<const F*>(P.mx)[k]);
            if (P.epilogue == RWKV_EPI_RESIDUAL || P.epilogue == RWKV_EPI_MUL_RESIDUAL) auxv = ldc<F>(P.aux, k);
            if (P.epilogue == RWKV_EPI_MUL_RESIDUAL) aux2v = ldc<F>(P.aux2, k);
        }
        const float val = fmaf(rxk, s, fmaf(rxk * 128.5f, txr, fmaf(mxk, tx, txmy)));
        store_epilogue_with<F>(P, k, val, auxv, aux2v);
    }
    if constexpr (kExch) {
        // The last CTA of the launch to finish forwards the launch's results to the other ranks:
        // wide stores over NVLink, ONE system-scope fence, then the arrival words.  (A fence per
        // CTA, with every CTA storing its own columns remotely, cost ~12 us per launch.)
        __shared__ unsigned s_last;
        __syncthreads();
        if (tid == 0) {
            __threadfence();                     // this CTA's results, before it reports
            s_last = atomicAdd(ex.done_counter, 1u) == gridDim.x - 1 ? 1u : 0u;
        }
        __syncthreads();
        if (s_last) {
            __threadfence();                     // every CTA's results are visible here
            for (int zz = 0; zz < kMaxProblems && b.panel_start[zz] < b.panel_start[kMaxProblems]; ++zz) {
                if (b.panel_start[zz + 1] == b.panel_start[zz]) continue;
                const Problem& Q = b.p[zz];
                const int es = Q.epilogue == RWKV_EPI_STORE_F32 ? 4 : int(sizeof(F));
                const long long bytes = (long long)Q.M * es;
                const char* src = static_cast<const char*>(Q.y);
                const bool vec = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
                const long long nv = vec ? bytes >> 4 : 0;
                for (int pr = 0; pr < ex.n_peers; ++pr) {
                    char* dst = static_cast<char*>(ex.peer_y[zz][pr]);          // same offset on the peer: same alignment
                    for (long long i = tid; i < nv; i += kThreads)
                        reinterpret_cast<uint4*>(dst)[i] = __ldcg(reinterpret_cast<const uint4*>(src) + i);
                    for (long long o = nv * 16 + 2 * tid; o < bytes; o += 2 * kThreads)
                        *reinterpret_cast<uint16_t*>(dst + o) = __ldcg(reinterpret_cast<const uint16_t*>(src + o));
                }
            }
            __syncthreads();
            if (tid == 0) {
                atomicExch(ex.done_counter, 0u);
                __threadfence_system();          // the forwarded results, system-wide, before the words
                const unsigned sig = ex.signal_seq + (ex.seq_base ? __ldcg(ex.seq_base) : 0u);
                for (int pr = 0; pr < ex.n_peers; ++pr)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ex.peer_arrived[pr]), "r"(sig) : "memory");
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ex.arrived + ex.rank), "r"(sig) : "memory");
            }
        }
    }
    cluster.sync();                              // nobody leaves while its shared memory is being read
    MM8_STAMP(b.trace_id, blockIdx.x, 6);
    MM8_STAMP(b.trace_id, blockIdx.x, 7);
}

int g_cluster_size = 0;       // 0 = automatic, -1 = off, else forced (1, 2, 4 or 8)
int g_cluster_pw = 0;         // 0 = automatic, else forced panel width (multiple of 16)
// tuning table: launches whose matrices have `cols` output columns in all are planned for `clusters`
struct PlanEntry { long long cols; int clusters; };
PlanEntry g_plan[16];
int g_plan_n = 0;

// Clusters of `S` CTAs (256 threads, `smem` bytes each) that can be resident at once on the
// current device; 0 if the query fails.  Asked once per (device, S).
template <typename K>
static inline int cluster_slots(K kern, int S, int smem, int build) {
    static int cache[64][2][kMaxClusterSize + 1] = {};         // per device and build (the two builds share a function type)
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 0; }
    build = build ? 1 : 0;
    if (cache[dev][build][S] != 0) return cache[dev][build][S] > 0 ? cache[dev][build][S] : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(S) * 64u);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = size_t(smem);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = unsigned(S);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = -1; }
    cache[dev][build][S] = n;
    return n > 0 ? n : 0;
}

// Launch the validated problems of `plan_b` (mm8_plan filled them in) on the cluster kernel.
// RWKV_ERR_UNSUPPORTED: this batch is not eligible and the caller should use the ticket kernel.
static inline int mm8_cluster_launch(const Batch& plan_b, int count, int dtype, int mode, const Exchange* exch, bool wide_hint,
                                     cudaStream_t st) {
    if (g_cluster_size < 0) return RWKV_ERR_UNSUPPORTED;
    ClusterBatch cb;
    memset(&cb, 0, sizeof(cb));
    int min_n = INT32_MAX, max_n = 0;
    long long total_cols = 0;
    for (int i = 0; i < count; ++i) {
        cb.p[i] = plan_b.p[i];
        if (cb.p[i].N < min_n) min_n = cb.p[i].N;
        if (cb.p[i].N > max_n) max_n = cb.p[i].N;
        total_cols += cb.p[i].M;
        // the LayerNorm prologue fetches the previous token's vector in 16-byte pieces
        if (cb.p[i].prologue == RWKV_PRO_LN_MIX && cb.p[i].mode != 2 && reinterpret_cast<uintptr_t>(cb.p[i].p2) % 16 != 0)
            return RWKV_ERR_UNSUPPORTED;
    }
    for (int i = count; i < kMaxProblems; ++i) cb.p[i] = cb.p[0];
    // K-splits: 8 when every CTA still gets a few hundred rows, fewer for short matrices.
    int S = g_cluster_size > 0 ? g_cluster_size : kMaxClusterSize;
    if (S != 1 && S != 2 && S != 4 && S != 8) return RWKV_ERR_UNSUPPORTED;
    if (g_cluster_size == 0) while (S > 1 && min_n < S * 64) S >>= 1;
    const int rows_needed = ((max_n + S - 1) / S + 7) & ~7;
    if (rows_needed > kWideRowsPerCta) return RWKV_ERR_UNSUPPORTED;
    // more than 2048 rows per CTA (20480 in-features): the build with the larger x' buffer, fp16 / integer only.
    // `wide_hint` asks for that build although this launch would fit the other one: launches that alternate
    // between the two builds (different shared-memory footprints) lose their overlap (14B shape: 241 tok/s
    // alternating, 305 with the wide build throughout), so a model with such a matrix asks for it everywhere.
    const bool wide = (rows_needed > kMaxRowsPerCta || wide_hint) && dtype == RWKV_F16 && mode == 2;
    if (rows_needed > kMaxRowsPerCta && !wide) return RWKV_ERR_UNSUPPORTED;
    if ((exch != nullptr || wide) && (dtype != RWKV_F16 || mode != 2)) return RWKV_ERR_UNSUPPORTED;
    constexpr int RN = kMaxRowsPerCta, RW = kWideRowsPerCta;
    void (*kern)(ClusterBatch, NoExchange) = nullptr;
    void (*kern_x)(ClusterBatch, Exchange) = wide ? mm8_cluster_kernel<__half, 2, Exchange, RW> : mm8_cluster_kernel<__half, 2, Exchange, RN>;
    if (wide) kern = mm8_cluster_kernel<__half, 2, NoExchange, RW>;
    else if (dtype == RWKV_F16) kern = mode == 2 ? mm8_cluster_kernel<__half, 2, NoExchange, RN> : mode == 1 ? mm8_cluster_kernel<__half, 1, NoExchange, RN> : mm8_cluster_kernel<__half, 0, NoExchange, RN>;
    else kern = mode == 2 ? mm8_cluster_kernel<float, 2, NoExchange, RN> : mode == 1 ? mm8_cluster_kernel<float, 1, NoExchange, RN> : mm8_cluster_kernel<float, 0, NoExchange, RN>;
    const int smem = wide ? cluster_smem<RW>() : cluster_smem<RN>();
    if ((exch ? cudaFuncSetAttribute(kern_x, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
              : cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) {
        cudaGetLastError();
        return RWKV_ERR_UNSUPPORTED;
    }
    int slots = exch ? cluster_slots(kern_x, S, smem, wide) : cluster_slots(kern, S, smem, wide);
    if (slots <= 0) return RWKV_ERR_UNSUPPORTED;
    // Plan for four fifths of the resident clusters (26 of 33): the slots left free let the next
    // launch's first clusters become resident, and fill their rings, while this one still streams
    // (7B shape: 487 -> 507 tok/s; 14B shape: -1 %).  A negative panel_width of
    // rwkv_mm8_one_set_cluster plans for that many clusters instead.
    {
        int planned = 0;
        for (int i = 0; i < g_plan_n; ++i) if (g_plan[i].cols == total_cols) planned = g_plan[i].clusters;
        if (planned > 0) { if (planned < slots) slots = planned; }
        else if (g_cluster_pw < 0) { if (-g_cluster_pw < slots) slots = -g_cluster_pw; }
        else if (g_cluster_pw == 0 && slots >= 10) slots = slots * 4 / 5;
    }

    // Panel width: the narrowest multiple of 16 columns with which one wave of clusters covers
    // every matrix of the launch.
    int pw = g_cluster_pw > 0 ? (g_cluster_pw + 15) / 16 * 16 : 16;
    if (pw > kMaxPanelCols) pw = kMaxPanelCols;
    if (g_cluster_pw <= 0) {
        long long guess = (total_cols + slots - 1) / slots;
        pw = int((guess + 15) / 16 * 16);
        if (pw < 16) pw = 16;
        for (; pw < kMaxPanelCols; pw += 16) {
            int panels = 0;
            for (int i = 0; i < count; ++i) panels += (cb.p[i].M + pw - 1) / pw;
            if (panels <= slots) break;
        }
        if (pw > kMaxPanelCols) pw = kMaxPanelCols;
    }
    cb.pw = pw;
    cb.S = S;
    cb.panel_start[0] = 0;
    for (int i = 0; i < kMaxProblems; ++i) {
        const int panels = i < count ? (cb.p[i].M + pw - 1) / pw : 0;
        cb.panel_start[i + 1] = cb.panel_start[i] + panels;
        if (i < count) {
            cb.p[i].rows_per_cta = ((cb.p[i].N + S - 1) / S + 7) & ~7;
            cb.p[i].splits = S;
        }
    }
    const long long ctas = (long long)cb.panel_start[kMaxProblems] * S;
    if (ctas > INT32_MAX) return RWKV_ERR_UNSUPPORTED;

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
    cb.trace_id = 0;
#ifdef RWKV_MM8_TRACE
    cb.trace_id = g_mm8_trace_next++;
#endif
    cudaError_t e = exch ? cudaLaunchKernelEx(&cfg, kern_x, cb, *exch) : cudaLaunchKernelEx(&cfg, kern, cb, NoExchange{0});
    if (e != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    return RWKV_OK;
}

}  // namespace

extern "C" void rwkv_mm8_one_set_plan(int64_t total_columns, int clusters) {
    for (int i = 0; i < g_plan_n; ++i)
        if (g_plan[i].cols == total_columns) { g_plan[i].clusters = clusters; return; }
    if (g_plan_n < 16) { g_plan[g_plan_n].cols = total_columns; g_plan[g_plan_n].clusters = clusters; ++g_plan_n; }
}

extern "C" void rwkv_mm8_one_set_cluster(int cluster_size, int panel_width) {
    g_cluster_size = cluster_size;
    g_cluster_pw = panel_width;
}
