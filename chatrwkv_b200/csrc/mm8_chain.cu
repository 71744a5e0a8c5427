// mm8 chain: a fixed list of dependent mm8_one launches (the att/ffn matmuls of every layer of
// one decode step) as ONE persistent cooperative kernel.
//
// Why: at batch 1 every matmul of a token is a 17-84 MB stream that takes 3-13 us at HBM
// speed, and a kernel boundary (drain, launch, first loads, split reduction) costs as much
// again.  Here the CTAs stay resident (two per SM), walk the list of launches ("phases")
// together and separate them by a grid barrier.  Nothing that can be known early waits for
// the barrier:
//   * the weight stream is never interrupted: while a CTA finishes phase p (reduction,
//     ticket, barrier, prologue of p+1) its cp.async ring already holds its first rows of
//     phase p+1;
//   * each CTA's description of phase p+2 (one record prepared by the host) and the per-row
//     constants of phase p+1 (scales, LayerNorm weights, mix factors, last token's state)
//     travel to shared memory with cp.async a phase ahead.
// After the barrier only what the previous phase produced is fetched: one round trip.  With
// the HBM saturated a dependent round trip costs ~3 us, so round trips, not bytes, are what
// the phase boundary is made of.
//
// Per phase the work split, the arithmetic, the prologues/epilogues and the deterministic
// split-K reduction are those of the single-launch kernel (mm8_one.cu).
//
// Waiting: the only wait is the grid barrier (a counter in global memory).  It is bounded:
// a CTA that does not see the barrier open within kSpinLimit polls raises the error word and
// every CTA then runs through the remaining phases without waiting, so the kernel always
// terminates; the host reads the error word with rwkv_mm8_chain_take_error.
#include <string.h>

#include "mm8_core.cuh"

namespace {

constexpr int kDepth = 4;
constexpr int kRing = ring_bytes(kDepth);            // 64 KB
constexpr int kRedBytes = kWarps * 512 * 4;          // 16 KB
// Staged per-row vectors of the prologue, laid out per tile as [nh half vectors][nf fp32
// vectors], each `cap` entries long (cap = rows of the tile rounded up to 32).  Bytes per row:
// PLAIN 2*2, LN_MIX 6*2, WKV4 2*2 + 5*4.  x' itself (fp32, up to 2048 rows) shares its 16 KB with
// the CTA reduction buffer: it is dead when the reduction starts.
constexpr int kStageBytes = 20480;
constexpr int kRowsPlain = 2048, kRowsLnMix = 1024, kRowsWkv4 = 832;
constexpr int kEpiBytes = 4 * 1024;                  // rx, mx, aux, aux2 of the panel's columns (fp16)
constexpr unsigned kSpinLimit = 1u << 22;

// Everything CTA c needs to know about phase p; written by the host, copied in 16-byte chunks.
struct __align__(16) CtaPhase {
    Problem P;
    float* partial;
    float* sums;
    unsigned* counters;
    int active, panel, split, col0, j0, nrows, lpr, pad0;
};
constexpr int kRecBytes = (sizeof(CtaPhase) + 15) / 16 * 16;
constexpr int kRecChunks = kRecBytes / 16;
constexpr int kSmemBytes = kRing + kRedBytes + kStageBytes + kEpiBytes + 3 * kRecBytes;

struct Tile {           // this thread's view of one phase's tile
    const uint8_t* wp;
    long long step;
    int nrows, sub, valid, rpp, ngroups, base;
};

__device__ __forceinline__ void make_tile(const CtaPhase& r, int tid, int base, Tile& t) {
    t.base = base;
    t.ngroups = 0;
    t.valid = 0;
    t.nrows = 0;
    t.sub = 0;
    t.rpp = 8;
    t.wp = nullptr;
    t.step = 0;
    if (!r.active) return;
    const int lane = tid & 31, warp = tid >> 5;
    const int lpr = r.lpr, rpw = 32 / lpr;
    t.rpp = kWarps * rpw;
    t.nrows = r.nrows;
    t.sub = warp * rpw + lane / lpr;
    const int c = r.col0 + (lane % lpr) * 16;
    t.valid = min(16, r.P.M - c);
    const int nsteps = (t.nrows + t.rpp - 1) / t.rpp;
    t.ngroups = (nsteps + kGroup - 1) / kGroup;
    t.wp = r.P.w + (long long)(r.j0 + t.sub) * r.P.w_stride + c;
    t.step = (long long)t.rpp * r.P.w_stride;
}

// Commit one ring group: rows [g*kGroup, g*kGroup + kGroup) of tile t (nothing if g is past its
// end); always exactly one commit, so that commit counts stay uniform.
__device__ __forceinline__ void issue(const Tile& t, int g, uint32_t slot0) {
    if (g < t.ngroups && t.valid > 0) {
#pragma unroll
        for (int u = 0; u < kGroup; ++u) {
            const int i = g * kGroup + u;
            if (t.sub + i * t.rpp < t.nrows)
                cp_async16(slot0 + (((t.base + g) % kDepth) * kGroup + u) * (kThreads * 16), t.wp + i * t.step);
        }
    }
    cp_async_commit();
}

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

__device__ __forceinline__ int row_cap(const CtaPhase& r) { return (r.nrows + 31) & ~31; }

// Stage the per-row vectors of a tile that no phase of this launch writes (scales, LayerNorm
// weight and bias, mix factors, the previous token's state).  No commit here: the copies join
// the next ring group.
__device__ __forceinline__ void stage_rows(const CtaPhase& r, uint32_t stage, int tid) {
    if (!r.active) return;
    const Problem& P = r.P;
    const int cap = row_cap(r);
    const uint32_t hbase = stage;
    const int npairs = (r.nrows + 1) / 2;
    const __half* hsrc[6] = {static_cast<const __half*>(P.ry), static_cast<const __half*>(P.my),
                             nullptr, nullptr, nullptr, nullptr};
    if (P.prologue == RWKV_PRO_LN_MIX) {
        hsrc[2] = static_cast<const __half*>(P.p0);
        hsrc[3] = static_cast<const __half*>(P.p1);
        if (P.mode != 2) {
            hsrc[4] = static_cast<const __half*>(P.p2);
            hsrc[5] = static_cast<const __half*>(P.p3);
        }
    }
    for (int q = tid; q < npairs; q += kThreads) {
#pragma unroll
        for (int a = 0; a < 6; ++a)
            if (hsrc[a]) cp_async4(hbase + a * (cap * 2) + q * 4, hsrc[a] + r.j0 + 2 * q);
    }
    if (P.prologue == RWKV_PRO_WKV4) {
        const uint32_t fbase = hbase + 2 * (cap * 2);
        const float* fsrc[5] = {P.f0, P.f1, P.f2, P.f3, P.f4};
        for (int j = tid; j < r.nrows; j += kThreads) {
#pragma unroll
            for (int a = 0; a < 5; ++a) cp_async4(fbase + a * (cap * 4) + j * 4, fsrc[a] + r.j0 + j);
        }
    }
}

// Stage what the epilogue of this tile's panel will need: rx, mx (constants) and aux, aux2
// (written by earlier phases, so L2-coherent 16-byte copies).  One chunk per thread.
__device__ __forceinline__ void stage_epilogue(const CtaPhase& r, uint32_t epi, int tid) {
    if (!r.active) return;
    const Problem& P = r.P;
    const int arr = tid >> 6, ch = tid & 63;             // 4 arrays x 64 chunks of 8 halfs
    const int k = r.col0 + ch * 8;
    if (ch * 8 >= r.lpr * 16 || k + 8 > P.M) return;     // ragged panel ends are loaded directly
    const void* src = arr == 0 ? P.rx : arr == 1 ? P.mx : arr == 2 ? P.aux : P.aux2;
    if (src == nullptr) return;
    cp_async16(epi + arr * 1024 + ch * 16, static_cast<const __half*>(src) + k);
}

__device__ __forceinline__ void fetch_record(const uint8_t* src, uint32_t dst, int tid) {
    if (tid < kRecChunks) cp_async16(dst + tid * 16, src + tid * 16);
}

// Bounded grid barrier.  Returns false once the error word is set (by this or another CTA).
__device__ __forceinline__ bool grid_barrier(unsigned* bar, unsigned target, unsigned* err, int* sh_ok) {
    __syncthreads();
    if (threadIdx.x == 0) {
        int ok = 1;
        __threadfence();
        atomicAdd(bar, 1u);
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
// prologue done, main loop done, partials written, ticket taken, epilogue done.
template <bool PACKED>
__global__ void __launch_bounds__(kThreads, 2) mm8_chain_kernel(const uint8_t* __restrict__ records, int n_phases,
                                                                unsigned* bar, unsigned* err,
                                                                unsigned long long* trace) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;                                                    // [slot][thread] 16 B
    float* red = reinterpret_cast<float*>(smem + kRing);                     // [row group][position]
    float* xs = red;                                                         // x' of this tile's rows
    uint8_t* stage = smem + kRing + kRedBytes;                               // staged per-row vectors
    uint8_t* epi = stage + kStageBytes;                                      // staged epilogue operands
    uint8_t* recs = epi + kEpiBytes;                                         // 3 phase records
    __shared__ float ssum[kWarps][3];
    __shared__ float sh8[kWarps];
    __shared__ unsigned s_ticket;
    __shared__ int s_ok;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x;
    const unsigned G = gridDim.x;
    const uint32_t slot0 = (uint32_t)__cvta_generic_to_shared(ring) + tid * 16;
    const uint32_t stage_s = (uint32_t)__cvta_generic_to_shared(stage);
    const uint32_t epi_s = (uint32_t)__cvta_generic_to_shared(epi);
    const uint32_t recs_s = (uint32_t)__cvta_generic_to_shared(recs);
    typedef __half F;
    auto rec_src = [&](int ph) { return records + ((long long)ph * G + cta) * kRecBytes; };
    auto rec = [&](int ph) -> const CtaPhase& { return *reinterpret_cast<const CtaPhase*>(recs + (ph % 3) * kRecBytes); };

    // records of phases 0 and 1 synchronously; phase p fetches the record of phase p+2 into the
    // slot that phase p-1 no longer needs
    for (int i = tid; i < 2 * kRecChunks; i += kThreads) {
        const int ph = i / kRecChunks, ch = i % kRecChunks;
        if (ph < n_phases)
            reinterpret_cast<uint4*>(recs + ph * kRecBytes)[ch] = __ldg(reinterpret_cast<const uint4*>(rec_src(ph)) + ch);
    }
    __syncthreads();
    Tile cur, nxt;
    make_tile(rec(0), tid, 0, cur);
    stage_rows(rec(0), stage_s, tid);
#pragma unroll
    for (int g = 0; g < kDepth; ++g) issue(cur, g, slot0);       // positions 0..kDepth-1 of phase 0
    bool healthy = true;

    for (int ph = 0; ph < n_phases; ++ph) {
        const bool tr = trace != nullptr && cta == 0 && tid == 0;
        if (tr) trace[ph * 8 + 0] = gtime();
        // Everything older than the last kDepth-1 commits has landed: this tile's staged rows,
        // ring position 0 and the record of phase ph+1.  The barrier's __syncthreads publishes it.
        cp_async_wait<kDepth - 1>();
        if (ph > 0 && healthy) healthy = grid_barrier(bar, unsigned(ph) * G, err, &s_ok);
        else __syncthreads();
        if (tr) trace[ph * 8 + 1] = gtime();

        const CtaPhase& R = rec(ph);
        const bool has_next = ph + 1 < n_phases;
        if (has_next) make_tile(rec(ph + 1), tid, (cur.base + cur.ngroups) % kDepth, nxt);
        else { nxt.ngroups = 0; nxt.valid = 0; nxt.nrows = 0; nxt.base = 0; nxt.sub = 0; nxt.rpp = 8; }

        int nxt_issued = 0;
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;

        if (R.active) {
            const Problem& P = R.P;
            const int cap = row_cap(R);
            const __half* h_ry = reinterpret_cast<const __half*>(stage);
            const __half* h_my = h_ry + cap;
            const bool writer = R.panel == 0;
            float sx = 0.f, sxr = 0.f, sxmy = 0.f;
            // ---- prologue: only what the previous phase wrote is loaded from global memory ----
            if (P.prologue == RWKV_PRO_LN_MIX) {
                const __half* h_lw = h_ry + 2 * cap;
                const __half* h_lb = h_ry + 3 * cap;
                const __half* h_sx = h_ry + 4 * cap;
                const __half* h_mix = h_ry + 5 * cap;
                const int nvec = P.N / 8;
                uint4 xv4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int v = tid + i * kThreads;
                    xv4[i] = v < nvec ? __ldcg(reinterpret_cast<const uint4*>(P.x) + v) : make_uint4(0, 0, 0, 0);
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
                const float rstd = rsqrtf(block_sum256(q, sh8) / float(P.N) + 1e-5f);
                // the rows of this tile are computed by whichever thread holds them in registers
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int j8 = (tid + i * kThreads) * 8;
                    if (j8 >= R.j0 && j8 < R.j0 + R.nrows) {
                        const __half* hx = reinterpret_cast<const __half*>(&xv4[i]);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const int l = j8 + e - R.j0;
                            const float xx = r16((__half2float(hx[e]) - mean) * rstd * __half2float(h_lw[l]) + __half2float(h_lb[l]));
                            if (writer && P.q0) static_cast<__half*>(P.q0)[j8 + e] = __float2half_rn(xx);
                            float xv = xx;
                            if (P.mode != 2) {
                                const float sxv = __half2float(h_sx[l]), mv = __half2float(h_mix[l]);
                                xv = P.mode == 0 ? r16(r16(xx * mv) + r16(sxv * r16(1.0f - mv))) : r16(xx + r16(r16(sxv - xx) * mv));
                            }
                            const float xp = xv * __half2float(h_ry[l]);
                            xs[l] = xp;
                            sx += xv;
                            sxr += xp;
                            sxmy = fmaf(xv, __half2float(h_my[l]), sxmy);
                        }
                    }
                }
            } else {
                const float* f_td = reinterpret_cast<const float*>(h_ry + 2 * cap);
                for (int l = tid; l < R.nrows; l += kThreads) {
                    const int j = R.j0 + l;
                    float xv;
                    if (P.prologue == RWKV_PRO_PLAIN) {
                        xv = ldc<F>(P.x, j);
                    } else {        // RWKV_PRO_WKV4 (pkg/model.py:1041-1055)
                        const float r = ldc<__half>(P.x, j), kk = ldc<__half>(P.p0, j), vv = ldc<__half>(P.p1, j);
                        const float td = f_td[l], tf = f_td[cap + l];
                        const float a = f_td[2 * cap + l], bq = f_td[3 * cap + l], p0 = f_td[4 * cap + l];
                        float ww = tf + kk;
                        float p = fmaxf(p0, ww);
                        float e1 = expf(p0 - p), e2 = expf(ww - p);
                        const float wkv = r16((e1 * a + e2 * vv) / (e1 * bq + e2));
                        if (writer) {
                            ww = td + p0;
                            p = fmaxf(ww, kk);
                            e1 = expf(ww - p); e2 = expf(kk - p);
                            P.g0[j] = e1 * a + e2 * vv;
                            P.g1[j] = e1 * bq + e2;
                            P.g2[j] = p;
                        }
                        xv = r16(r * wkv);
                    }
                    const float xp = xv * __half2float(h_ry[l]);
                    xs[l] = xp;
                    sx += xv;
                    sxr += xp;
                    sxmy = fmaf(xv, __half2float(h_my[l]), sxmy);
                }
            }
            sx = warp_sum(sx); sxr = warp_sum(sxr); sxmy = warp_sum(sxmy);
            if (lane == 0) { ssum[warp][0] = sx; ssum[warp][1] = sxr; ssum[warp][2] = sxmy; }
        }
        __syncthreads();                         // x' complete; the staged rows are no longer read
        if (tr) trace[ph * 8 + 2] = gtime();
        // On their way while this phase streams (they join the next ring commit): the next tile's
        // per-row constants, what this tile's epilogue will read, and the record of the phase
        // after the next.
        if (has_next) stage_rows(rec(ph + 1), stage_s, tid);
        stage_epilogue(R, epi_s, tid);
        if (ph + 2 < n_phases) fetch_record(rec_src(ph + 2), recs_s + ((ph + 2) % 3) * kRecBytes, tid);

        // ---- main loop: drain group g, then commit stream position g + kDepth ----
        for (int g = 0; g < cur.ngroups; ++g) {
            cp_async_wait<kDepth - 1>();
            uint4 v[kGroup];
#pragma unroll
            for (int u = 0; u < kGroup; ++u)
                v[u] = *reinterpret_cast<const uint4*>(ring + tid * 16 + (((cur.base + g) % kDepth) * kGroup + u) * (kThreads * 16));
            if (cur.valid > 0) {
#pragma unroll
                for (int u = 0; u < kGroup; ++u) {
                    const int r = cur.sub + (g * kGroup + u) * cur.rpp;
                    if (r < cur.nrows) fma16<PACKED>(acc, v[u], xs[r]);
                }
            }
            if (g + kDepth < cur.ngroups) issue(cur, g + kDepth, slot0);
            else issue(nxt, nxt_issued++, slot0);
        }
        // the next phase always starts with exactly kDepth commits of its own
        while (nxt_issued < kDepth) issue(nxt, nxt_issued++, slot0);
        if (tr) trace[ph * 8 + 3] = gtime();

        if (R.active) {
            const Problem& P = R.P;
            const int LPR = R.lpr, PW = LPR * 16, RPP = cur.rpp;
            // ---- CTA reduce (the buffer also held x': every thread must be out of the main loop).
            // The wait makes this thread's share of the staged epilogue operands land: they went
            // out with the first commit of this phase, and at least three commits followed.
            cp_async_wait<kDepth - 1>();
            __syncthreads();
            {
                const int rg = cur.sub, l = lane % LPR;
#pragma unroll
                for (int i = 0; i < 16; ++i) red[rg * PW + i * LPR + l] = acc[i];
            }
            __syncthreads();
            float* part = R.partial + P.partial_off + (long long)R.split * P.m_pad + R.col0;
            for (int p = tid; p < PW; p += kThreads) {
                float s = 0.f;
                for (int rg = 0; rg < RPP; ++rg) s += red[rg * PW + p];
                part[p] = s;
            }
            float* sums = R.sums + (long long)(P.counter_off + R.panel) * kMaxSplit * 4;
            if (tid < 3) {
                float s = 0.f;
#pragma unroll
                for (int w8 = 0; w8 < kWarps; ++w8) s += ssum[w8][tid];
                sums[R.split * 4 + tid] = s;
            }
            if (tr) trace[ph * 8 + 4] = gtime();
            // ---- ticket: one fence by the thread that takes it, after the CTA barrier ----
            __syncthreads();
            if (tid == 0) {
                __threadfence();
                s_ticket = atomicAdd(&R.counters[P.counter_off + R.panel], 1u);
            }
            __syncthreads();
            if (tr) trace[ph * 8 + 5] = gtime();
            if (s_ticket == unsigned(P.splits - 1)) {
                __threadfence();
                if (tid == 0) R.counters[P.counter_off + R.panel] = 0u;
                const int S = P.splits;
                float t0 = 0.f, t1 = 0.f, t2 = 0.f;
                if (tid < S) {
                    t0 = __ldcg(sums + tid * 4 + 0);
                    t1 = __ldcg(sums + tid * 4 + 1);
                    t2 = __ldcg(sums + tid * 4 + 2);
                }
                float sacc[2] = {0.f, 0.f};
                const float* pbase = R.partial + P.partial_off + R.col0 + tid;
                const int ppt = (PW + kThreads - 1) / kThreads;
                if (tid < PW) {
                    // all loads of a batch are independent: 16 splits (x 2 positions) in flight
                    for (int sp = 0; sp < S; sp += 16) {
                        float a[16][2];
#pragma unroll
                        for (int u = 0; u < 16; ++u)
#pragma unroll
                            for (int h = 0; h < 2; ++h)
                                a[u][h] = (sp + u < S && h < ppt) ? __ldcg(pbase + (long long)(sp + u) * P.m_pad + h * kThreads) : 0.f;
#pragma unroll
                        for (int u = 0; u < 16; ++u) { sacc[0] += a[u][0]; sacc[1] += a[u][1]; }
                    }
                }
                const float tx = block_sum256(t0, sh8);
                const float txr = block_sum256(t1, sh8);
                const float txmy = block_sum256(t2, sh8);
                const __half* e_rx = reinterpret_cast<const __half*>(epi);
                const __half* e_mx = e_rx + 512;
                const __half* e_aux = e_rx + 1024;
                const __half* e_aux2 = e_rx + 1536;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int p = tid + h * kThreads;
                    const int kk = (p % LPR) * 16 + p / LPR, k = R.col0 + kk;
                    if (h < ppt && p < PW && k < P.M) {
                        float rxk, mxk, auxv = 0.f, aux2v = 0.f;
                        if (R.col0 + (kk | 7) < P.M) {       // this 8-column chunk was staged
                            rxk = __half2float(e_rx[kk]); mxk = __half2float(e_mx[kk]);
                            if (P.aux) auxv = __half2float(e_aux[kk]);
                            if (P.aux2) aux2v = __half2float(e_aux2[kk]);
                        } else {
                            rxk = __half2float(static_cast<const F*>(P.rx)[k]); mxk = __half2float(static_cast<const F*>(P.mx)[k]);
                            if (P.aux) auxv = ldc<F>(P.aux, k);
                            if (P.aux2) aux2v = ldc<F>(P.aux2, k);
                        }
                        const float val = fmaf(rxk, sacc[h], fmaf(rxk * 128.5f, txr, fmaf(mxk, tx, txmy)));
                        store_epilogue_with<F>(P, k, val, auxv, aux2v);
                    }
                }
            }
        }
        if (tr) trace[ph * 8 + 6] = gtime();
        cur = nxt;
    }
    cp_async_wait<0>();
}

}  // namespace

extern "C" int rwkv_mm8_chain_ctas(void) { return 2 * rwkv_sm_count(); }

extern "C" size_t rwkv_mm8_chain_table_bytes(int n_launches, int n_ctas) {
    return (n_launches > 0 && n_ctas > 0) ? size_t(n_launches) * size_t(n_ctas) * size_t(kRecBytes) : 0;
}

extern "C" int rwkv_mm8_chain_plan(const rwkv_mm8_problem* problems, const int32_t* counts, int n_launches,
                                   int dtype, int n_ctas, void* workspace, size_t workspace_bytes,
                                   void* table_out, size_t table_bytes) {
    RWKV_CHECK_ARG(problems && counts && n_launches >= 1 && table_out && n_ctas >= 1);
    RWKV_CHECK_ARG(dtype == RWKV_F16);
    if (table_bytes < rwkv_mm8_chain_table_bytes(n_launches, n_ctas)) return RWKV_ERR_INVALID_ARG;
    uint8_t* out = static_cast<uint8_t*>(table_out);
    int off = 0;
    for (int l = 0; l < n_launches; ++l) {
        LaunchPlan plan;
        static const int max_rows[3] = {kRowsPlain, kRowsLnMix, kRowsWkv4};
        const int rc = mm8_plan(problems + off, counts[l], dtype, workspace, workspace_bytes, n_ctas, true, 0, 0,
                                max_rows, plan);
        if (rc != RWKV_OK) return rc;
        if (!plan.aligned) return RWKV_ERR_ALIGNMENT;     // the chain has no byte-load path
        int tiles = 0;
        for (int z = 0; z < counts[l]; ++z) {
            const Problem& P = plan.b.p[z];
            if (P.N % 2 != 0 || (P.epilogue != RWKV_EPI_STORE && P.epilogue != RWKV_EPI_SIGMOID &&
                                 P.epilogue != RWKV_EPI_RELU_SQ && P.epilogue != RWKV_EPI_RESIDUAL &&
                                 P.epilogue != RWKV_EPI_MUL_RESIDUAL)) return RWKV_ERR_UNSUPPORTED;
            tiles += ((P.M + plan.pw - 1) / plan.pw) * P.splits;
        }
        if (tiles > n_ctas) return RWKV_ERR_UNSUPPORTED;
        int c = 0;
        for (int z = 0; z < counts[l]; ++z) {
            const Problem& P = plan.b.p[z];
            const int panels = (P.M + plan.pw - 1) / plan.pw;
            for (int t = 0; t < panels * P.splits; ++t, ++c) {
                CtaPhase r;
                memset(&r, 0, sizeof(r));
                r.P = P;
                r.partial = plan.b.partial; r.sums = plan.b.sums; r.counters = plan.b.counters;
                r.active = 1;
                r.panel = t % panels; r.split = t / panels;
                r.col0 = r.panel * plan.pw;
                r.j0 = r.split * P.rows_per_cta;
                r.nrows = (P.N < r.j0 + P.rows_per_cta ? P.N : r.j0 + P.rows_per_cta) - r.j0;
                r.lpr = plan.pw / 16;
                memcpy(out + (size_t(l) * n_ctas + c) * kRecBytes, &r, sizeof(r));
            }
        }
        for (; c < n_ctas; ++c) memset(out + (size_t(l) * n_ctas + c) * kRecBytes, 0, kRecBytes);
        off += counts[l];
    }
    return RWKV_OK;
}

extern "C" int rwkv_mm8_chain_run(const void* table_device, int n_launches, int n_ctas, void* workspace,
                                  void* trace, void* stream) {
    RWKV_CHECK_ARG(table_device && n_launches >= 1 && workspace && n_ctas >= 1);
    RWKV_CHECK_ALIGN(table_device, 16);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto kern = mm8_chain_kernel<true>;
    const int smem = kSmemBytes;                         // ~104 KB: two CTAs per SM, never three
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
            cudaGetLastError();
            return RWKV_ERR_LAUNCH;
        }
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem) != cudaSuccess) {
            cudaGetLastError();
            return RWKV_ERR_LAUNCH;
        }
        if (per_sm * rwkv_sm_count() < n_ctas) return RWKV_ERR_UNSUPPORTED;   // the grid must be co-resident
        configured = true;
    }
    unsigned* words = static_cast<unsigned*>(workspace);
    unsigned* bar = words + (kCounterBytes / 4 - 2);
    unsigned* err = words + (kCounterBytes / 4 - 1);
    if (cudaMemsetAsync(bar, 0, sizeof(unsigned), st) != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    const uint8_t* table = static_cast<const uint8_t*>(table_device);
    unsigned long long* tr = static_cast<unsigned long long*>(trace);
    void* args[] = {(void*)&table, (void*)&n_launches, (void*)&bar, (void*)&err, (void*)&tr};
    // Cooperative launch: the runtime guarantees that all CTAs are resident, which the grid
    // barrier relies on.
    cudaError_t e = cudaLaunchCooperativeKernel((const void*)kern, dim3(n_ctas), dim3(kThreads), args, size_t(smem), st);
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
