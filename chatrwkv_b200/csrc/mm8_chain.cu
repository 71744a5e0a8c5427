// mm8 chain: a fixed list of dependent mm8_one launches (the att/ffn matmuls of every layer of
// one decode step) as ONE persistent cooperative kernel of thread-block clusters.
//
// Why: at batch 1 every matmul of a token is a 17-84 MB stream that takes 3-13 us at HBM
// speed, and a kernel boundary costs as much again: the next kernel's CTAs only become
// resident as the previous one's clusters leave, so they start their streams at different
// times and with empty rings.  Here the clusters stay resident (8 CTAs each, two CTAs per
// SM), walk the list of launches ("phases") together and separate them by a grid barrier:
//   * the weight stream never stops: while a CTA reduces phase p, waits at the barrier and
//     runs the prologue of phase p+1, its cp.async ring already fills with its first rows of
//     phase p+1 (16 rows per thread, 64 KB per CTA);
//   * every model constant of phase p+1 (scales of the CTA's rows and columns, LayerNorm
//     weights, mix factors, decay), the cluster's description of phase p+2 and L2 prefetches
//     of the previous token's state are issued during the stream of phase p;
//   * after the barrier only what the previous phase produced is fetched: one trip to L2.
// A phase's K-splits are the 8 CTAs of a cluster; they add their column sums through
// distributed shared memory in rank order (bit-reproducible), exactly as in the single-launch
// cluster kernel (mm8_cluster.cuh), whose arithmetic, prologues and epilogues this file shares.
//
// Waiting: cluster barriers (hardware, among co-scheduled CTAs) and ONE software wait, the
// grid barrier: a counter in global memory that one thread per cluster bumps and one thread
// per CTA polls.  It is bounded: a CTA that does not see the barrier open within kSpinLimit
// polls raises the error word and every CTA then runs through the remaining phases without
// waiting, so the kernel always terminates; the host reads the error word with
// rwkv_mm8_chain_take_error.  The launch is cooperative, so all clusters are resident.
#include <cooperative_groups.h>
#include <string.h>

#include "mm8_core.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int kDepth = 4;
constexpr int kS = 8;                                // cluster size = K-splits of every phase
constexpr int kRing = ring_bytes(kDepth);            // 64 KB
constexpr int kStageBuf = 16384;                     // ry, my (2048 rows, fp16) + 8 KB prologue constants
constexpr int kExtraOff = 8192;
constexpr int kExtraRows = 1024;                     // rows whose LayerNorm / WKV constants fit the 8 KB
constexpr int kEpiCols = 512;                        // columns a CTA finishes
constexpr int kEpiConst = 2 * kEpiCols * 2;          // rx, mx (fp16) of one phase
constexpr int kMaxPanel = 2048;                      // the column sums share the 8 KB of x'
constexpr int kChainRows = 2048;                     // rows per CTA (the stage buffers are laid out for this)
constexpr unsigned kSpinLimit = 1u << 22;

// What a cluster does in one phase; written by the host, copied in 16-byte chunks.
struct __align__(16) ClusterPhase {
    Problem P;
    int active, col0, ncols, pad0;
};
constexpr int kRecBytes = (sizeof(ClusterPhase) + 15) / 16 * 16;
constexpr int kRecChunks = kRecBytes / 16;
// ring | stage[2] | rx,mx [2] | aux, aux2 | 3 records
constexpr int kOffStage = kRing;
constexpr int kOffEpiConst = kOffStage + 2 * kStageBuf;
constexpr int kOffAux = kOffEpiConst + 2 * kEpiConst;
constexpr int kOffRecs = kOffAux + 2 * kEpiCols * 2;
constexpr int kSmemBytes = kOffRecs + 3 * kRecBytes;
static_assert(kSmemBytes <= 104 * 1024, "shared-memory plan exceeds two CTAs per SM");

struct Tile {           // this thread's share of one phase's weight stream
    const uint8_t* wp;
    long long step;
    int nrows, sub, rpp, ngroups, base, active;
};

struct Geo {            // where this CTA works in a phase
    int j0, nrows, cpr, rpp, PWc, per, kc0, kc1;
};

__device__ __forceinline__ Geo geometry(const ClusterPhase& r, int rank) {
    Geo g;
    g.j0 = rank * r.P.rows_per_cta;
    g.nrows = r.active ? max(0, min(r.P.N, g.j0 + r.P.rows_per_cta) - g.j0) : 0;
    g.cpr = max(1, (r.ncols + 15) >> 4);
    g.rpp = kThreads / g.cpr;
    g.PWc = g.cpr * 16;
    g.per = ((r.ncols + kS - 1) / kS + 7) & ~7;
    g.kc0 = min(r.ncols, rank * g.per);
    g.kc1 = min(r.ncols, g.kc0 + g.per);
    if (!r.active) { g.kc0 = g.kc1 = 0; }
    return g;
}

__device__ __forceinline__ void make_tile(const ClusterPhase& r, const Geo& g, int tid, int base, Tile& t) {
    t.base = base;
    t.sub = tid / g.cpr;
    const int ch = tid - t.sub * g.cpr;
    t.rpp = g.rpp;
    t.active = r.active && t.sub < g.rpp;
    t.nrows = g.nrows;
    const int nsteps = (g.nrows + g.rpp - 1) / g.rpp;
    t.ngroups = r.active ? (nsteps + kGroup - 1) / kGroup : 0;
    t.wp = r.active ? r.P.w + (long long)(g.j0 + t.sub) * r.P.w_stride + r.col0 + ch * 16 : nullptr;
    t.step = (long long)g.rpp * r.P.w_stride;
}

// Commit one ring group: rows [g*kGroup, g*kGroup + kGroup) of tile t (nothing if g is past its
// end); always exactly one commit, so that commit counts stay uniform.
__device__ __forceinline__ void issue(const Tile& t, int g, uint32_t slot0) {
    if (t.active && g < t.ngroups) {
#pragma unroll
        for (int u = 0; u < kGroup; ++u) {
            const int i = g * kGroup + u;
            if (t.sub + i * t.rpp < t.nrows)
                cp_async16(slot0 + (((t.base + g) % kDepth) * kGroup + u) * (kThreads * 16), t.wp + i * t.step);
        }
    }
    cp_async_commit();
}

// Model constants of a phase for this CTA: scales of its rows, prologue constants, scales of the
// columns it finishes.  No commit here: the copies join the next ring commit.
__device__ __forceinline__ void stage_constants(const ClusterPhase& r, const Geo& g, uint8_t* stage, uint8_t* epic, int tid) {
    if (!r.active) return;
    const Problem& P = r.P;
    stage_vec<2>(stage, P.ry, g.j0, g.nrows, tid);
    stage_vec<2>(stage + 2 * kChainRows, P.my, g.j0, g.nrows, tid);
    if (g.nrows <= kExtraRows) {
        uint8_t* ex = stage + kExtraOff;
        if (P.prologue == RWKV_PRO_LN_MIX) {
            stage_vec<2>(ex, P.p0, g.j0, g.nrows, tid);
            stage_vec<2>(ex + 2 * kExtraRows, P.p1, g.j0, g.nrows, tid);
            if (P.mode != 2) stage_vec<2>(ex + 4 * kExtraRows, P.p3, g.j0, g.nrows, tid);
        } else if (P.prologue == RWKV_PRO_WKV4) {
            stage_vec<4>(ex, P.f0, g.j0, g.nrows, tid);
            stage_vec<4>(ex + 4 * kExtraRows, P.f1, g.j0, g.nrows, tid);
        }
    }
    stage_vec<2>(epic, P.rx, r.col0 + g.kc0, g.kc1 - g.kc0, tid);
    stage_vec<2>(epic + 2 * kEpiCols, P.mx, r.col0 + g.kc0, g.kc1 - g.kc0, tid);
    // the previous token's state of these rows: toward L2 (a hint; the loads follow the barrier)
    if (P.prologue == RWKV_PRO_LN_MIX && P.mode != 2) l2_prefetch<2>(P.p2, g.j0, g.nrows, tid);
    if (P.prologue == RWKV_PRO_WKV4) {
        l2_prefetch<4>(P.f2, g.j0, g.nrows, tid);
        l2_prefetch<4>(P.f3, g.j0, g.nrows, tid);
        l2_prefetch<4>(P.f4, g.j0, g.nrows, tid);
    }
}

__device__ __forceinline__ void fetch_record(const uint8_t* src, uint32_t dst, int tid) {
    if (tid < kRecChunks) cp_async16(dst + tid * 16, src + tid * 16);
}

// Bounded grid barrier over clusters.  The caller has made this cluster's stores visible
// (__threadfence by the storing threads, then a cluster barrier); `leader` = rank 0 of the
// cluster.  Returns false once the error word is set (by this or another CTA).
__device__ __forceinline__ bool grid_barrier(unsigned* bar, unsigned target, unsigned* err, bool leader, int* sh_ok) {
    if (threadIdx.x == 0) {
        int ok = 1;
        if (leader) {
            __threadfence();
            atomicAdd(bar, 1u);
        }
        unsigned it = 0;
        while (true) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar) : "memory");
            if (v >= target) break;
            if ((++it & 1023u) == 0) {
                unsigned e;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(e) : "l"(err) : "memory");
                if (e != 0 || it >= kSpinLimit) { atomicExch(err, 1u); ok = 0; break; }
            }
        }
        __threadfence();
        *sh_ok = ok;
    }
    __syncthreads();
    return *sh_ok != 0;
}

__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// trace (optional): [phase][8] nanosecond stamps of CTA 0 -- phase start, barrier passed,
// prologue done, main loop done, column sums sent, cluster reduced, epilogue done.
__global__ void __launch_bounds__(kThreads, 2) mm8_chain_kernel(const uint8_t* __restrict__ records, int n_phases,
                                                                int n_clusters, unsigned* bar, unsigned* err,
                                                                unsigned long long* trace) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;                                                    // [slot][thread] 16 B
    uint8_t* recs = smem + kOffRecs;                                         // 3 phase records
    __shared__ float xs[kChainRows];                                         // x' of this CTA's rows; later its column sums
    __shared__ float ssum[kWarps][3];
    __shared__ float sh8[kWarps];
    __shared__ float tot3[4];
    __shared__ float all3[4];
    __shared__ int s_ok;
    typedef __half F;

    cg::cluster_group cluster = cg::this_cluster();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rank = int(cluster.block_rank());
    const int cid = int(blockIdx.x) / kS;
    const uint32_t slot0 = (uint32_t)__cvta_generic_to_shared(ring) + tid * 16;
    const uint32_t recs_s = (uint32_t)__cvta_generic_to_shared(recs);
    auto rec_src = [&](int ph) { return records + ((long long)ph * n_clusters + cid) * kRecBytes; };
    auto rec = [&](int ph) -> const ClusterPhase& { return *reinterpret_cast<const ClusterPhase*>(recs + (ph % 3) * kRecBytes); };
    auto stage_of = [&](int ph) { return smem + kOffStage + (ph & 1) * kStageBuf; };
    auto epic_of = [&](int ph) { return smem + kOffEpiConst + (ph & 1) * kEpiConst; };
    F* s_aux = reinterpret_cast<F*>(smem + kOffAux);
    F* s_aux2 = s_aux + kEpiCols;

    // records of phases 0 and 1 synchronously; phase p fetches the record of phase p+2 into the
    // slot that phase p-1 no longer needs
    for (int i = tid; i < 2 * kRecChunks; i += kThreads) {
        const int ph = i / kRecChunks, ch = i % kRecChunks;
        if (ph < n_phases)
            reinterpret_cast<uint4*>(recs + ph * kRecBytes)[ch] = __ldg(reinterpret_cast<const uint4*>(rec_src(ph)) + ch);
    }
    __syncthreads();
    Geo gcur = geometry(rec(0), rank), gnxt = gcur;
    Tile cur, nxt;
    make_tile(rec(0), gcur, tid, 0, cur);
    stage_constants(rec(0), gcur, stage_of(0), epic_of(0), tid);     // joins the commit of ring group 0
#pragma unroll
    for (int g = 0; g < kDepth; ++g) issue(cur, g, slot0);            // positions 0..kDepth-1 of phase 0
    bool healthy = true;

    for (int ph = 0; ph < n_phases; ++ph) {
        const bool tr = trace != nullptr && blockIdx.x == 0 && tid == 0;
        if (tr) trace[ph * 8 + 0] = gtime();
        // Everything older than the last kDepth-1 commits has landed: this phase's staged constants,
        // ring position 0 and the record of phase ph+1.  The barrier's __syncthreads publishes it.
        cp_async_wait<kDepth - 1>();
        if (ph > 0 && healthy) healthy = grid_barrier(bar, unsigned(ph) * unsigned(n_clusters), err, rank == 0, &s_ok);
        else __syncthreads();
        if (tr) trace[ph * 8 + 1] = gtime();

        const ClusterPhase& R = rec(ph);
        const Problem& P = R.P;
        const Geo G = gcur;
        const bool has_next = ph + 1 < n_phases;
        if (has_next) {
            gnxt = geometry(rec(ph + 1), rank);
            make_tile(rec(ph + 1), gnxt, tid, (cur.base + cur.ngroups) % kDepth, nxt);
        } else {
            nxt.active = 0; nxt.ngroups = 0; nxt.nrows = 0; nxt.base = 0; nxt.sub = 0; nxt.rpp = 8; nxt.wp = nullptr; nxt.step = 0;
        }
        uint8_t* stage = stage_of(ph);
        const F* s_ry = reinterpret_cast<const F*>(stage);
        const F* s_my = s_ry + kChainRows;
        const uint8_t* s_extra = stage + kExtraOff;
        const F* s_rx = reinterpret_cast<const F*>(epic_of(ph));
        const F* s_mx = s_rx + kEpiCols;
        const bool extra_staged = G.nrows <= kExtraRows;
        const int j0 = G.j0, j1 = G.j0 + G.nrows, nrows = G.nrows;
        const bool writer = R.col0 == 0;

        // ---- prologue: one trip to L2 for what earlier phases wrote, then x' = x * ry ---------
        float sx = 0.f, sxr = 0.f, sxmy = 0.f;
        if (R.active && P.prologue == RWKV_PRO_LN_MIX) {
            uint4 xv4[4], sv4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int j8 = (tid + i * kThreads) * 8;
                xv4[i] = j8 < P.N ? __ldcg(reinterpret_cast<const uint4*>(P.x) + (j8 >> 3)) : make_uint4(0, 0, 0, 0);
                sv4[i] = (P.mode != 2 && j8 >= j0 && j8 < j1) ? __ldcg(reinterpret_cast<const uint4*>(P.p2) + (j8 >> 3))
                                                              : make_uint4(0, 0, 0, 0);
            }
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __half2* h = reinterpret_cast<const __half2*>(&xv4[i]);
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h[e]); s += f.x + f.y; }
            }
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
            const __half* lb = extra_staged ? reinterpret_cast<const __half*>(s_extra + 2 * kExtraRows) : static_cast<const __half*>(P.p1) + j0;
            const __half* mixv = P.mode == 2 ? nullptr
                               : extra_staged ? reinterpret_cast<const __half*>(s_extra + 4 * kExtraRows) : static_cast<const __half*>(P.p3) + j0;
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
                        const float xp = xv * __half2float(s_ry[l]);
                        xs[l] = xp;
                        sx += xv;
                        sxr += xp;
                        sxmy = fmaf(xv, __half2float(s_my[l]), sxmy);
                    }
                }
            }
        } else if (R.active && P.prologue == RWKV_PRO_WKV4) {     // pkg/model.py:1041-1055
            const float* tdv = extra_staged ? reinterpret_cast<const float*>(s_extra) : P.f0 + j0;
            const float* tfv = extra_staged ? reinterpret_cast<const float*>(s_extra + 4 * kExtraRows) : P.f1 + j0;
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
                const float xp = xv * __half2float(s_ry[l]);
                xs[l] = xp;
                sx += xv;
                sxr += xp;
                sxmy = fmaf(xv, __half2float(s_my[l]), sxmy);
            }
        } else if (R.active) {
            constexpr int RPT = kChainRows / kThreads;
            float xr[RPT];
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                const int l = tid + i * kThreads;
                xr[i] = l < nrows ? ldc<F>(P.x, j0 + l) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                const int l = tid + i * kThreads;
                if (l < nrows) {
                    const float xv = xr[i];
                    const float xp = xv * __half2float(s_ry[l]);
                    xs[l] = xp;
                    sx += xv;
                    sxr += xp;
                    sxmy = fmaf(xv, __half2float(s_my[l]), sxmy);
                }
            }
        }
        sx = warp_sum(sx); sxr = warp_sum(sxr); sxmy = warp_sum(sxmy);
        if (lane == 0) { ssum[warp][0] = sx; ssum[warp][1] = sxr; ssum[warp][2] = sxmy; }
        __syncthreads();                         // x' complete; this phase's staged rows are no longer read
        if (tr) trace[ph * 8 + 2] = gtime();
        // On their way while this phase streams (they join the next ring commit): what this phase's
        // epilogue adds or multiplies, the next phase's constants, and the record after the next.
        if (R.active) {
            if (P.epilogue == RWKV_EPI_RESIDUAL || P.epilogue == RWKV_EPI_MUL_RESIDUAL)
                stage_vec<2>(reinterpret_cast<uint8_t*>(s_aux), P.aux, R.col0 + G.kc0, G.kc1 - G.kc0, tid);
            if (P.epilogue == RWKV_EPI_MUL_RESIDUAL)
                stage_vec<2>(reinterpret_cast<uint8_t*>(s_aux2), P.aux2, R.col0 + G.kc0, G.kc1 - G.kc0, tid);
        }
        if (has_next) stage_constants(rec(ph + 1), gnxt, stage_of(ph + 1), epic_of(ph + 1), tid);
        if (ph + 2 < n_phases) fetch_record(rec_src(ph + 2), recs_s + ((ph + 2) % 3) * kRecBytes, tid);

        // ---- main loop: drain group g, then commit stream position g + kDepth ----------------
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
        int nxt_issued = 0;
        for (int g = 0; g < cur.ngroups; ++g) {
            cp_async_wait<kDepth - 1>();
            uint4 v[kGroup];
#pragma unroll
            for (int u = 0; u < kGroup; ++u)
                v[u] = *reinterpret_cast<const uint4*>(ring + tid * 16 + (((cur.base + g) % kDepth) * kGroup + u) * (kThreads * 16));
            if (cur.active) {
#pragma unroll
                for (int u = 0; u < kGroup; ++u) {
                    const int r = cur.sub + (g * kGroup + u) * cur.rpp;
                    if (r < cur.nrows) fma16<true>(acc, v[u], xs[r]);
                }
            }
            if (g + kDepth < cur.ngroups) issue(cur, g + kDepth, slot0);
            else issue(nxt, nxt_issued++, slot0);
        }
        // the next phase always starts with exactly kDepth commits of its own
        while (nxt_issued < kDepth) issue(nxt, nxt_issued++, slot0);
        if (tr) trace[ph * 8 + 3] = gtime();

        // ---- CTA reduce (in the stage buffer of this phase, dead since the prologue).  The wait
        // makes this thread's share of the staged epilogue operands land: they went out with the
        // first commit after the prologue, and kDepth commits followed.
        cp_async_wait<kDepth - 1>();
        __syncthreads();                         // every thread is out of the main loop: x' is dead too
        float* red = reinterpret_cast<float*>(stage);            // [rpp][PWc] <= 16 KB
        float* cs = xs;                                          // [PWc] column sums of this CTA
        if (cur.active) {
            const int ch = tid - cur.sub * G.cpr;
#pragma unroll
            for (int i = 0; i < 16; ++i) red[cur.sub * G.PWc + ch * 16 + ((i + ch) & 15)] = acc[i];
        }
        __syncthreads();
        if (R.active) {
            for (int kk = tid; kk < G.PWc; kk += kThreads) {
                const int pos = (kk & ~15) + (((kk & 15) + (kk >> 4)) & 15);
                float s = 0.f;
                for (int rg = 0; rg < G.rpp; ++rg) s += red[rg * G.PWc + pos];
                cs[kk] = s;
            }
            if (tid < 3) {
                float s = 0.f;
#pragma unroll
                for (int w8 = 0; w8 < kWarps; ++w8) s += ssum[w8][tid];
                tot3[tid] = s;
            }
        }
        if (tr) trace[ph * 8 + 4] = gtime();
        cluster.sync();                          // every CTA's cs / tot3 are complete and visible
        if (tr) trace[ph * 8 + 5] = gtime();

        // ---- cluster reduce through distributed shared memory, in rank order ------------------
        if (R.active) {
            if (warp == 0) {
                float v0 = 0.f, v1 = 0.f, v2 = 0.f;
                if (lane < kS) {
                    const float* rt = cluster.map_shared_rank(tot3, lane);
                    v0 = rt[0]; v1 = rt[1]; v2 = rt[2];
                }
                float t0 = 0.f, t1 = 0.f, t2 = 0.f;
#pragma unroll
                for (int q = 0; q < kS; ++q) {
                    t0 += __shfl_sync(0xffffffffu, v0, q);
                    t1 += __shfl_sync(0xffffffffu, v1, q);
                    t2 += __shfl_sync(0xffffffffu, v2, q);
                }
                if (lane == 0) { all3[0] = t0; all3[1] = t1; all3[2] = t2; }
            }
            __syncthreads();
            const float tx = all3[0], txr = all3[1], txmy = all3[2];
            for (int kk = G.kc0 + tid; kk < G.kc1; kk += kThreads) {
                float a[kS];
#pragma unroll
                for (int q = 0; q < kS; ++q) a[q] = cluster.map_shared_rank(cs, q)[kk];
                float s = 0.f;
#pragma unroll
                for (int q = 0; q < kS; ++q) s += a[q];
                const int k = R.col0 + kk, e = kk - G.kc0;
                const float rxk = __half2float(s_rx[e]), mxk = __half2float(s_mx[e]);
                float auxv = 0.f, aux2v = 0.f;
                if (P.epilogue == RWKV_EPI_RESIDUAL || P.epilogue == RWKV_EPI_MUL_RESIDUAL) auxv = __half2float(s_aux[e]);
                if (P.epilogue == RWKV_EPI_MUL_RESIDUAL) aux2v = __half2float(s_aux2[e]);
                const float val = fmaf(rxk, s, fmaf(rxk * 128.5f, txr, fmaf(mxk, tx, txmy)));
                store_epilogue_with<F>(P, k, val, auxv, aux2v);
            }
        }
        __threadfence();                         // this thread's results, before the cluster reports at the grid barrier
        cluster.sync();                          // peers are done reading this CTA's sums; the cluster's results are out
        if (tr) trace[ph * 8 + 6] = gtime();
        cur = nxt;
        gcur = gnxt;
    }
    cp_async_wait<0>();
}

}  // namespace

namespace {

// Clusters of 8 CTAs of the chain kernel that fit the current device at once (0: query failed).
int chain_clusters() {
    static int cache[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 0; }
    if (cache[dev] != 0) return cache[dev] > 0 ? cache[dev] : 0;
    int n = -1;
    if (cudaFuncSetAttribute(mm8_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 104 * 1024) == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(kS * 64);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = 104 * 1024;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = kS;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, mm8_chain_kernel, &cfg) != cudaSuccess || n <= 0) n = -1;
    }
    cudaGetLastError();
    cache[dev] = n;
    return n > 0 ? n : 0;
}

}  // namespace

// CTAs of a chain launch on the current device: 8 per resident cluster.
extern "C" int rwkv_mm8_chain_ctas(void) { return kS * chain_clusters(); }

extern "C" size_t rwkv_mm8_chain_table_bytes(int n_launches, int n_ctas) {
    return (n_launches > 0 && n_ctas >= kS) ? size_t(n_launches) * size_t(n_ctas / kS) * size_t(kRecBytes) : 0;
}

extern "C" int rwkv_mm8_chain_plan(const rwkv_mm8_problem* problems, const int32_t* counts, int n_launches,
                                   int dtype, int n_ctas, void* workspace, size_t workspace_bytes,
                                   void* table_out, size_t table_bytes) {
    RWKV_CHECK_ARG(problems && counts && n_launches >= 1 && table_out && n_ctas >= kS && n_ctas % kS == 0);
    RWKV_CHECK_ARG(dtype == RWKV_F16);
    if (table_bytes < rwkv_mm8_chain_table_bytes(n_launches, n_ctas)) return RWKV_ERR_INVALID_ARG;
    const int C = n_ctas / kS;
    uint8_t* out = static_cast<uint8_t*>(table_out);
    int off = 0;
    for (int l = 0; l < n_launches; ++l) {
        LaunchPlan plan;
        static const int max_rows[3] = {kMaxRowsPerCta, kMaxRowsPerCta, kMaxRowsPerCta};
        const int count = counts[l];
        const int rc = mm8_plan(problems + off, count, dtype, workspace, workspace_bytes, n_ctas, false, 0, 0, max_rows, plan);
        if (rc != RWKV_OK) return rc;
        if (!plan.aligned) return RWKV_ERR_ALIGNMENT;     // the chain has no byte-load path
        long long total_cols = 0;
        for (int z = 0; z < count; ++z) {
            Problem& P = plan.b.p[z];
            if (P.epilogue != RWKV_EPI_STORE && P.epilogue != RWKV_EPI_SIGMOID && P.epilogue != RWKV_EPI_RELU_SQ &&
                P.epilogue != RWKV_EPI_RESIDUAL && P.epilogue != RWKV_EPI_MUL_RESIDUAL && P.epilogue != RWKV_EPI_SILU)
                return RWKV_ERR_UNSUPPORTED;
            P.rows_per_cta = ((P.N + kS - 1) / kS + 7) & ~7;
            P.splits = kS;
            if (P.rows_per_cta > kChainRows) return RWKV_ERR_UNSUPPORTED;
            if (P.prologue == RWKV_PRO_LN_MIX && P.mode != 2 && reinterpret_cast<uintptr_t>(P.p2) % 16 != 0) return RWKV_ERR_ALIGNMENT;
            total_cols += P.M;
        }
        // panel width: the narrowest multiple of 16 columns with which the clusters cover the launch
        int pw = int(((total_cols + C - 1) / C + 15) / 16 * 16);
        if (pw < 16) pw = 16;
        for (;; pw += 16) {
            int panels = 0;
            for (int z = 0; z < count; ++z) panels += (plan.b.p[z].M + pw - 1) / pw;
            if (panels <= C) break;
            if (pw >= kMaxPanel) return RWKV_ERR_UNSUPPORTED;
        }
        if (pw > kMaxPanel || (((pw + kS - 1) / kS + 7) & ~7) > kEpiCols) return RWKV_ERR_UNSUPPORTED;
        int c = 0;
        for (int z = 0; z < count; ++z) {
            const Problem& P = plan.b.p[z];
            const int panels = (P.M + pw - 1) / pw;
            for (int t = 0; t < panels; ++t, ++c) {
                ClusterPhase r;
                memset(&r, 0, sizeof(r));
                r.P = P;
                r.active = 1;
                r.col0 = t * pw;
                r.ncols = P.M - r.col0 < pw ? P.M - r.col0 : pw;
                memcpy(out + (size_t(l) * C + c) * kRecBytes, &r, sizeof(r));
            }
        }
        for (; c < C; ++c) memset(out + (size_t(l) * C + c) * kRecBytes, 0, kRecBytes);
        off += count;
    }
    return RWKV_OK;
}

extern "C" int rwkv_mm8_chain_run(const void* table_device, int n_launches, int n_ctas, void* workspace,
                                  void* trace, void* stream) {
    RWKV_CHECK_ARG(table_device && n_launches >= 1 && workspace && n_ctas >= kS && n_ctas % kS == 0);
    RWKV_CHECK_ALIGN(table_device, 16);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int resident = chain_clusters();
    if (resident <= 0 || n_ctas / kS > resident) return RWKV_ERR_UNSUPPORTED;   // the grid must be co-resident
    unsigned* words = static_cast<unsigned*>(workspace);
    unsigned* bar = words + (kCounterBytes / 4 - 2);
    unsigned* err = words + (kCounterBytes / 4 - 1);
    if (cudaMemsetAsync(bar, 0, sizeof(unsigned), st) != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    const uint8_t* table = static_cast<const uint8_t*>(table_device);
    unsigned long long* tr = static_cast<unsigned long long*>(trace);
    int n_clusters = n_ctas / kS;
    // Cooperative launch of clusters: the runtime guarantees that every CTA is resident, which
    // the grid barrier relies on.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(n_ctas));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = 104 * 1024;       // the plan needs kSmemBytes; the size also keeps two CTAs per SM
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeCooperative;
    attr[1].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, mm8_chain_kernel, table, n_launches, n_clusters, bar, err, tr);
    if (e != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    return RWKV_OK;
}

extern "C" int rwkv_mm8_chain_take_error(void* workspace, void* stream, int* error_out) {
    RWKV_CHECK_ARG(workspace != nullptr && error_out != nullptr);
    unsigned* flag = static_cast<unsigned*>(workspace) + (kCounterBytes / 4 - 1);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned v = 0;
    if (cudaMemcpyAsync(&v, flag, sizeof(v), cudaMemcpyDeviceToHost, st) != cudaSuccess) return RWKV_ERR_LAUNCH;
    if (cudaStreamSynchronize(st) != cudaSuccess) return RWKV_ERR_LAUNCH;
    if (v != 0 && cudaMemsetAsync(flag, 0, sizeof(v), st) != cudaSuccess) return RWKV_ERR_LAUNCH;
    *error_out = int(v);
    return RWKV_OK;
}
