// mm8_seq on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
//
//   y[t,n] = rx[n] * sum_k x'[t,k] (w[k,n] - 128) + rx[n]*128.5*SXR[t] + mx[n]*SX[t] + SXMY[t]
//
// with x' = x*ry, SX = sum_k x, SXR = sum_k x', SXMY = sum_k x*my (per row t): the same
// factorisation as mm8_one.  The contraction runs as fp16 x fp16 -> fp32 UMMA:
//   * (w - 128) is exact in fp16 and is produced on the fly: producer threads read uint8 rows
//     of W, transpose 8x8 byte blocks in registers and write fp16 core matrices (K-major,
//     no swizzle) into the B tile;
//   * x' (an fp32 product) is split into hi = fp16(x') and lo = fp16(x' - hi) by a small
//     preparation kernel; both halves are multiplied into the same accumulator, so the sum
//     carries ~22 bits of x' and matches the fp32 CUDA-core kernel to rounding.
//
// CTA = 128 (rows of x) x 256 (columns of W) output tile, K in blocks of 64, 3 stages.
//   warps 0-15 producers: fetch W rows four K blocks ahead into registers (8 k x 4 columns per thread and
//              K block) and convert them into the B tile.  Then epilogue: tcgen05.ld of their
//              32 TMEM lanes (warp % 4) x 64 columns (warp / 4), affine epilogue, fp16 stores
//   warp 16    TMEM allocation; lane 0 issues tcgen05.mma and tcgen05.commit
//   warp 17    lane 0 starts the bulk copies of the A tiles (the preparation kernel stores them as
//              ready-made 16 KB operand images)
// Synchronisation is by mbarriers only.  Every wait is bounded: on give-up the CTA raises an
// error word, skips the rest of its work, frees its tensor memory and returns.
// Launches with an even number of row tiles and no K split run the CTA-pair form (template PAIR = 2): two
// CTAs of a cluster share one 256 x 256 UMMA (cta_group::2), each converting half of the B tile.
#include "common.cuh"
#include "seq_epi.cuh"
#include <algorithm>
#include <cstdio>

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 3;
constexpr int kProducers = 512;
constexpr int kProdWarps = kProducers / 32;
constexpr int kThreadsTc = kProducers + 64;              // + the MMA warp and the warp that starts the A copies
constexpr int kWAhead = 4;                               // K blocks of W held in registers
constexpr int kTileBytes = 128 * BK * 2;                 // 16 KB: one 128 x 64 fp16 operand tile
constexpr uint32_t kSBO_B = (BK / 8) * 128 + 16;         // B: 8-row groups 16 bytes further apart, so that the
                                                         // 32 lanes that each store one core matrix of a
                                                         // different group hit different shared-memory banks
constexpr int kBTileBytes = (BN / 8) * kSBO_B;           // 32.5 KB
constexpr int kStageBytes = 2 * kTileBytes + kBTileBytes;   // A_hi, A_lo, B
constexpr int kSmemTc = STAGES * kStageBytes + 1024;     // + barriers, TMEM address
// The CTA-pair form (two row tiles of one column tile as a cluster of two CTAs, tcgen05 cta_group::2): each CTA
// converts and stores only its half of the B tile (128 columns), which the pair's tensor cores share; 4 stages.
constexpr int STAGES2 = 4;
constexpr int kStageBytes2 = 2 * kTileBytes + kBTileBytes / 2;
constexpr int kSmemTc2 = STAGES2 * kStageBytes2 + 1024;
constexpr uint32_t kLBO = 128;                           // bytes between core matrices along K
constexpr uint32_t kSBO = (BK / 8) * 128;                // A: bytes between 8-row groups
constexpr unsigned kWaitLimit = 1u << 22;

// Optional timeline of one CTA for tuning (compiled in only with -DRWKV_SEQ_TRACE): per K block the clock
// after the producers' wait, after their A copies were issued, after the B tile was stored, and on the MMA
// thread after its wait and after the issue.
#ifdef RWKV_SEQ_TRACE
constexpr int kTraceBlocks = 512;
__device__ long long g_seq_trace[2][kTraceBlocks][5];
#define SEQ_STAMP(kb, slot) do { if (traced && (kb) < kTraceBlocks) g_seq_trace[trace_row][kb][slot] = clock64(); } while (0)
#else
#define SEQ_STAMP(kb, slot) do { } while (0)
#endif

__device__ __forceinline__ uint32_t s2u(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (unsigned it = 0; it < kWaitLimit; ++it) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// one arrival on `bar` that also announces `bytes` of bulk-copy traffic to it
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// contiguous global -> shared bulk copy (both addresses 16-byte aligned, bytes % 16 == 0) that reports to `bar`
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"((uint64_t)__cvta_generic_to_global(src)), "r"(bytes), "r"(bar) : "memory");
}

// Shared-memory matrix descriptor: K-major, no swizzle, core matrices of 8 rows x 16 bytes.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);         // start address
    d |= (uint64_t)(kLBO >> 4) << 16;                    // leading (K) byte offset
    d |= (uint64_t)(sbo >> 4) << 32;                     // stride (M/N) byte offset
    d |= (uint64_t)1 << 46;                              // descriptor version of sm_100
    return d;                                            // layout type 0: no swizzle
}
// Instruction descriptor, kind::f16: fp16 A and B (both K-major), fp32 accumulator, M x N tile.
__device__ __forceinline__ uint32_t umma_idesc(int m, int n) {
    uint32_t d = 0;
    d |= 1u << 4;                       // accumulator format: f32
    d |= 0u << 7;                       // A: f16
    d |= 0u << 10;                      // B: f16
    d |= (uint32_t)(n >> 3) << 17;
    d |= (uint32_t)(m >> 4) << 24;
    return d;
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// ---- the same for a pair of CTAs (cta_group::2): issued by one thread of the pair's first CTA
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// `bar`: a shared::cluster address (this CTA's barrier, or the other CTA's through cluster_addr)
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_addr(uint32_t local, uint32_t rank) {     // the same offset in CTA `rank`
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity) {      // acquires what another CTA released
    for (unsigned it = 0; it < kWaitLimit; ++it) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- preparation: x' hi/lo split and the three row sums ---------------------------------------
// hi and lo are written in the order the GEMM consumes them: for every (128-row tile, K block of 64) one
// contiguous 16 KB image of the shared-memory operand tile (core matrices of 8 rows x 16 bytes, 128 bytes
// between K chunks, 1 KB between 8-row groups), so that the GEMM fetches a tile with one bulk copy.
// Columns from N up to the end of the last K block are zeros; rows from T up to the end of the last tile
// are left as they are (an output row depends on its own row of x' only, and those rows are not stored).
// One block = 8 rows (one group of core matrices) x one share of the K range (blockIdx.y, so that short
// sequences still fill the GPU); thread = (row, 16-byte chunk of 8 k).  Each share writes its own partial
// row sums, which the consumers add in share order.
template <typename F>
__device__ __forceinline__ void load8(const F* __restrict__ p, long long base, int k0, int N, bool vec, float (&out)[8]) {
    if (vec && k0 + 8 <= N) {
        if constexpr (sizeof(F) == 2) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(p + base + k0));
            const F* h = reinterpret_cast<const F*>(&v);
#pragma unroll
            for (int e = 0; e < 8; ++e) out[e] = to_f32<F>(h[e]);
            return;
        }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = (k0 + e < N) ? to_f32<F>(p[base + k0 + e]) : 0.f;
}

template <typename F>
__global__ void __launch_bounds__(256) mm8_seq_prep(int T, int N, int nkb, const F* __restrict__ x, long long x_stride,
                                                    const F* __restrict__ ry, const F* __restrict__ my, int vec_x, int vec_v,
                                                    int chunks_per, uint8_t* __restrict__ hi, uint8_t* __restrict__ lo,
                                                    float* __restrict__ sums) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int row = threadIdx.x & 7, cl = threadIdx.x >> 3;          // cl: 0..31
    const int t = blockIdx.x * 8 + row;
    const int rt = blockIdx.x >> 4, group = blockIdx.x & 15;         // 128-row tile, 8-row group within it
    __shared__ float sh[3][8][8];
    float sx = 0.f, sxr = 0.f, sxmy = 0.f;
    const int c_begin = blockIdx.y * chunks_per, c_end = min(nkb * 8, c_begin + chunks_per);
    for (int c = c_begin + cl; c < c_end; c += 32) {
        if (t >= T) break;
        const int k0 = c * 8;
        uint4 h4 = make_uint4(0, 0, 0, 0), l4 = make_uint4(0, 0, 0, 0);
        if (k0 < N) {
            float xv[8], rv[8], mv[8];
            load8<F>(x, (long long)t * x_stride, k0, N, vec_x != 0, xv);
            load8<F>(ry, 0, k0, N, vec_v != 0, rv);
            load8<F>(my, 0, k0, N, vec_v != 0, mv);
            __half* hh = reinterpret_cast<__half*>(&h4);
            __half* lh = reinterpret_cast<__half*>(&l4);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float xp = xv[e] * rv[e];
                sx += xv[e];
                sxr += xp;
                sxmy = fmaf(xv[e], mv[e], sxmy);
                hh[e] = __float2half_rn(xp);
                lh[e] = __float2half_rn(xp - __half2float(hh[e]));
            }
        }
        const size_t off = (size_t(rt) * nkb + (c >> 3)) * kTileBytes + group * kSBO + (c & 7) * kLBO + row * 16;
        *reinterpret_cast<uint4*>(hi + off) = h4;
        *reinterpret_cast<uint4*>(lo + off) = l4;
    }
    // row sums: lanes 8 and 16 apart hold the same row, then the 8 warps in order
    sx += __shfl_xor_sync(0xffffffffu, sx, 8);   sx += __shfl_xor_sync(0xffffffffu, sx, 16);
    sxr += __shfl_xor_sync(0xffffffffu, sxr, 8); sxr += __shfl_xor_sync(0xffffffffu, sxr, 16);
    sxmy += __shfl_xor_sync(0xffffffffu, sxmy, 8); sxmy += __shfl_xor_sync(0xffffffffu, sxmy, 16);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane < 8) { sh[0][warp][lane] = sx; sh[1][warp][lane] = sxr; sh[2][warp][lane] = sxmy; }
    __syncthreads();
    if (threadIdx.x < 24) {
        const int which = threadIdx.x >> 3, r = threadIdx.x & 7;
        float s = 0.f;
        for (int i = 0; i < 8; ++i) s += sh[which][i][r];
        if (blockIdx.x * 8 + r < T) sums[((size_t)blockIdx.y * T + blockIdx.x * 8 + r) * 4 + which] = s;
    }
}

// 8 bytes of one column (k = 0..7) -> 8 fp16 values (byte - 128), packed as a uint4
__device__ __forceinline__ uint4 bytes_to_half8(uint32_t lo4, uint32_t hi4) {
    const uint32_t magic = 0x64646464u;          // fp16 0x64xx = 1024 + xx
    const __half2 off = __floats2half2_rn(1152.f, 1152.f);
    uint32_t w[4] = {__byte_perm(lo4, magic, 0x5140), __byte_perm(lo4, magic, 0x5342),
                     __byte_perm(hi4, magic, 0x5140), __byte_perm(hi4, magic, 0x5342)};
    uint4 out;
    uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = __hsub2(*reinterpret_cast<__half2*>(&w[i]), off);
        o[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return out;
}

struct TcArgs {
    const uint8_t* hi; const uint8_t* lo;                     // fp16 operand tile images [row tile][K block][16 KB]
    const float* sums; int nsum;                              // [nsum][T][4]: partial SX, SXR, SXMY, added in order
    const uint8_t* w; long long w_stride;
    const void* mx; const void* rx;                           // [M] in the output dtype
    void* y; long long y_stride;
    int T, N, M;
    int vec_ok;                                               // y, rx, mx allow 16-byte accesses
    int single;                                               // 1: multiply fp16(x*ry) only (no low-order pass)
    unsigned* error_flag;
    // K split over blockIdx.z (launches of one row tile that would leave most SMs idle): CTA z takes K
    // blocks [z * kb_per, (z + 1) * kb_per) and writes its fp32 sums to partial[z][t][m_pad]
    int ksplit, kb_per, m_pad;
    float* partial;
    SeqEpi epi;
};

// PAIR = 1: one CTA per output tile.  PAIR = 2: the CTAs (x, 2j) and (x, 2j + 1) form a cluster and run ONE
// 256 x 256 UMMA per step (cta_group::2): CTA r holds its own 128 rows of A and columns [128 r, 128 r + 128) of
// the B tile, so the uint8 -> fp16 conversion, its shared-memory stores and the tensor cores' reads of B are
// halved per CTA (the shared-memory pipe was the limit of the one-CTA form).  The first CTA's MMA thread issues
// for both; the second CTA's MMA thread forwards "my stage is full" to it; tcgen05.commit frees the stage in both.
template <typename F, int PAIR>
__global__ void __launch_bounds__(kThreadsTc, 1) mm8_seq_tc_kernel(const TcArgs a) {
    asm volatile("griddepcontrol.launch_dependents;");
    constexpr int S = PAIR == 2 ? STAGES2 : STAGES;
    constexpr int SB = PAIR == 2 ? kStageBytes2 : kStageBytes;
    constexpr int NPW = PAIR == 2 ? kProdWarps / 2 : kProdWarps;      // warps that convert W (all 16 run the epilogue)
    const uint32_t crank = PAIR == 2 ? cluster_rank() : 0u;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // pair form: grid.x = 2 x column tiles, the CTAs (2c, y) and (2c + 1, y) are the cluster that owns row tiles 2y, 2y + 1
    const int row_tile = PAIR == 2 ? int(blockIdx.y) * 2 + int(blockIdx.x & 1) : int(blockIdx.y);
    const int n0 = (PAIR == 2 ? int(blockIdx.x >> 1) : int(blockIdx.x)) * BN, m0 = row_tile * BM;
    const int nkb_all = (a.N + BK - 1) / BK;
    const int kbase = a.ksplit > 1 ? int(blockIdx.z) * a.kb_per : 0;            // first K block of this CTA
    const int nkb = a.ksplit > 1 ? max(0, min(nkb_all, kbase + a.kb_per) - kbase) : nkb_all;
#ifdef RWKV_SEQ_TRACE
    const bool last_cta = blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1;
    const bool traced = (tid == 0 || tid == kProducers || tid == kProducers + 32) && blockIdx.z == 0 && ((blockIdx.x == 0 && blockIdx.y == 0) || last_cta);
    const int trace_row = last_cta ? 1 : 0;
#endif

    uint8_t* bars = smem + S * SB;
    const uint32_t full0 = s2u(bars), empty0 = full0 + S * 8, accum_bar = empty0 + S * 8;
    const uint32_t pfull0 = accum_bar + 8;               // pair form, first CTA: "the other CTA's stage is full"
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + (3 * S + 1) * 8);
    int* failed = reinterpret_cast<int*>(bars + (3 * S + 1) * 8 + 8);

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full0 + s * 8, NPW + 1);           // one arrival per producer warp (its B part is stored and fenced)
                                                         // + the thread that starts the A copies
            mbar_init(empty0 + s * 8, 1);                // tcgen05.commit
            mbar_init(pfull0 + s * 8, 1);
        }
        mbar_init(accum_bar, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kProdWarps) {                            // one warp (the same in both CTAs of a pair) allocates BN fp32 accumulator columns
        if constexpr (PAIR == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)), "r"(BN) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)), "r"(BN) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if constexpr (PAIR == 2) cluster_barrier();          // both CTAs' barriers exist before either one signals the other's
    else __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // Only what the preceding kernels wrote has to wait for them: the operand images and row sums of the preparation
    // kernel, the residual inputs, and the output itself.  The producers' whole main loop reads nothing but the
    // packed matrix, so it runs ahead of the wait (under programmatic dependent launch: while the preparation kernel
    // and the tail of the previous matmul are still at work).

    if (warp < kProdWarps) {
        // ================= producers =================
        const int cg = PAIR == 2 ? (tid & 31) : (tid & 63);      // B: 4 columns x 8 k-rows per thread
        const int rg = PAIR == 2 ? ((tid >> 5) & 7) : (tid >> 6);
        const int ncol = n0 + int(crank) * (BN / 2) + cg * 4;
        const bool col_ok = ncol < a.M;                  // M % 8 == 0 is a launch condition
        uint32_t wreg[kWAhead][8];                       // W rows of the next kWAhead K blocks
        auto load_w = [&](int kb, uint32_t (&dst)[8]) {
            const int k0 = (kbase + kb) * BK + rg * 8;
            const uint8_t* p = a.w + (long long)k0 * a.w_stride + ncol;
            if (col_ok && k0 + 8 <= a.N) {                   // all but the ragged edges: one add per row
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    dst[i] = __ldg(reinterpret_cast<const uint32_t*>(p));
                    p += a.w_stride;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    dst[i] = (col_ok && k0 + i < a.N) ? __ldg(reinterpret_cast<const uint32_t*>(p + (long long)i * a.w_stride))
                                                      : 0x80808080u;      // code 128 -> value 0
            }
        };
        const bool converts = warp < NPW;
#pragma unroll
        for (int u = 0; u < kWAhead; ++u)
            if (u < nkb && converts) load_w(u, wreg[u]);
        bool ok = true;
        int s = 0;                                           // stage of K block kb and the parity of its use
        uint32_t ph = 0;
        for (int kb0 = 0; kb0 < nkb && ok && converts; kb0 += kWAhead) {
#pragma unroll
            for (int u = 0; u < kWAhead; ++u) {
                const int kb = kb0 + u;
                if (kb >= nkb || !ok) continue;
                ok = mbar_wait(empty0 + s * 8, ph ^ 1);
                if (!ok) continue;
                SEQ_STAMP(kb, 0);
                uint8_t* stage = smem + s * SB;
                // B tile: transpose this thread's 8 (k) x 4 (columns) byte block, convert, store four
                // rows of one core matrix: column j holds k = 0..3 in lo4[j] and k = 4..7 in hi4[j]
                uint32_t lo4[4], hi4[4];
#pragma unroll
                for (int half = 0; half < 2; ++half) {       // k rows 0-3, 4-7
                    const uint32_t a0 = wreg[u][half * 4 + 0], a1 = wreg[u][half * 4 + 1];
                    const uint32_t a2 = wreg[u][half * 4 + 2], a3 = wreg[u][half * 4 + 3];
                    const uint32_t x00 = __byte_perm(a0, a1, 0x5140), x01 = __byte_perm(a2, a3, 0x5140);
                    const uint32_t x10 = __byte_perm(a0, a1, 0x7362), x11 = __byte_perm(a2, a3, 0x7362);
                    uint32_t* dstw = half ? hi4 : lo4;
                    dstw[0] = __byte_perm(x00, x01, 0x5410);
                    dstw[1] = __byte_perm(x00, x01, 0x7632);
                    dstw[2] = __byte_perm(x10, x11, 0x5410);
                    dstw[3] = __byte_perm(x10, x11, 0x7632);
                }
                if (kb + kWAhead < nkb) load_w(kb + kWAhead, wreg[u]);   // refill this register slot
                uint8_t* bt = stage + 2 * kTileBytes + (cg >> 1) * kSBO_B + rg * kLBO + (cg & 1) * 64;
#pragma unroll
                for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(bt + j * 16) = bytes_to_half8(lo4[j], hi4[j]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();                                // 512 arrivals per stage on one barrier word were the
                if (lane == 0) mbar_arrive(full0 + s * 8);   // kernel's limit (~1 us per K block): one per warp instead
                SEQ_STAMP(kb, 2);
                if (++s == S) { s = 0; ph ^= 1; }
            }
        }
        // ================= epilogue =================
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (ok) ok = mbar_wait(accum_bar, 0);
        if (!ok) atomicExch(failed, 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int quarter = warp & 3, cq = warp >> 2;        // TMEM lanes 32*quarter.., columns 64*cq..
            const int t = m0 + quarter * 32 + lane;
            float sx = 0.f, sxr = 0.f, sxmy = 0.f;
            if (t < a.T)
                for (int z = 0; z < a.nsum; ++z) {
                    const float* sp = a.sums + ((size_t)z * a.T + t) * 4;
                    sx += sp[0]; sxr += sp[1]; sxmy += sp[2];
                }
            const F* mx = static_cast<const F*>(a.mx);
            const F* rx = static_cast<const F*>(a.rx);
            F* yrow = static_cast<F*>(a.y) + (long long)t * a.y_stride;
#pragma unroll 1
            for (int c = cq * 2; c < cq * 2 + 2; ++c) {
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + c * 32;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                    "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (a.ksplit > 1) {
                    if (t < a.T) {               // raw fp32 sums of this K range; rwkv seq_reduce finishes them
                        float4* prow = reinterpret_cast<float4*>(a.partial + ((long long)blockIdx.z * a.T + t) * a.m_pad + n0 + c * 32);
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            prow[q] = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                                  __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                    }
                } else if (t < a.T) {
                    const int nb = n0 + c * 32;
                    if (a.vec_ok && nb + 32 <= a.M) {       // 4 x (8 columns: 16-byte loads of rx, mx, 16-byte store)
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint4 r4 = __ldg(reinterpret_cast<const uint4*>(rx + nb) + q);
                            const uint4 m4 = __ldg(reinterpret_cast<const uint4*>(mx + nb) + q);
                            const __half* rh = reinterpret_cast<const __half*>(&r4);
                            const __half* mh = reinterpret_cast<const __half*>(&m4);
                            uint4 o4, x4 = make_uint4(0, 0, 0, 0), z4 = make_uint4(0, 0, 0, 0);
                            if (a.epi.mode == RWKV_EPI_RESIDUAL || a.epi.mode == RWKV_EPI_MUL_RESIDUAL)
                                x4 = *(reinterpret_cast<const uint4*>(static_cast<const __half*>(a.epi.aux) + (long long)t * a.epi.aux_stride + nb) + q);
                            if (a.epi.mode == RWKV_EPI_MUL_RESIDUAL)
                                z4 = *(reinterpret_cast<const uint4*>(static_cast<const __half*>(a.epi.aux2) + (long long)t * a.epi.aux2_stride + nb) + q);
                            const __half* xh = reinterpret_cast<const __half*>(&x4);
                            const __half* zh = reinterpret_cast<const __half*>(&z4);
                            __half* oh = reinterpret_cast<__half*>(&o4);
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                const float rxn = __half2float(rh[e]);
                                const float val = fmaf(rxn, __uint_as_float(v[q * 8 + e]),
                                                       fmaf(rxn * 128.5f, sxr, fmaf(__half2float(mh[e]), sx, sxmy)));
                                oh[e] = seq_epilogue_with<__half>(a.epi.mode, a.epi.out_scale, val, __half2float(xh[e]), __half2float(zh[e]));
                            }
                            reinterpret_cast<uint4*>(yrow + nb)[q] = o4;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int n = nb + j;
                            if (n < a.M) {
                                const float rxn = to_f32<F>(rx[n]);
                                const float val = fmaf(rxn, __uint_as_float(v[j]), fmaf(rxn * 128.5f, sxr, fmaf(to_f32<F>(mx[n]), sx, sxmy)));
                                yrow[n] = seq_epilogue<F>(a.epi, t, n, val);
                            }
                        }
                    }
                }
            }
        }
    } else if (warp == kProdWarps + 1) {
        // ================= A tiles: one bulk copy each (hi, lo) of the 16 KB image the preparation kernel laid out
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool ok = true;
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % S;
                const uint32_t ph = (kb / S) & 1;
                ok = mbar_wait(empty0 + s * 8, ph ^ 1);
                if (!ok) break;
                const uint32_t a_hi = s2u(smem + s * SB), a_lo = a_hi + kTileBytes;
                const size_t src = (size_t(row_tile) * nkb_all + kbase + kb) * kTileBytes;
                mbar_arrive_expect_tx(full0 + s * 8, a.single ? kTileBytes : 2 * kTileBytes);
                bulk_g2s(a_hi, a.hi + src, kTileBytes, full0 + s * 8);
                if (!a.single) bulk_g2s(a_lo, a.lo + src, kTileBytes, full0 + s * 8);
                SEQ_STAMP(kb, 1);
            }
            if (!ok) atomicExch(failed, 1);
        }
    } else if (lane == 0 && crank == 0) {
        // ================= MMA issuer =================
        const uint32_t idesc = umma_idesc(BM * PAIR, BN);
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const int s = kb % S;
            const uint32_t ph = (kb / S) & 1;
            ok = mbar_wait(full0 + s * 8, ph);
            if (PAIR == 2 && ok) ok = mbar_wait_cluster(pfull0 + s * 8, ph);
            if (!ok) break;
            SEQ_STAMP(kb, 3);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            const uint32_t a_hi = s2u(smem + s * SB), a_lo = a_hi + kTileBytes, b_t = a_hi + 2 * kTileBytes;
#pragma unroll
            for (int j = 0; j < BK / 16; ++j) {          // one UMMA consumes K = 16: two core matrices
                const uint64_t bd = umma_desc(b_t + j * 2 * kLBO, kSBO_B);
                if constexpr (PAIR == 2) {
                    umma_f16_pair(tmem_base, umma_desc(a_hi + j * 2 * kLBO, kSBO), bd, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                    if (!a.single) umma_f16_pair(tmem_base, umma_desc(a_lo + j * 2 * kLBO, kSBO), bd, idesc, 1u);
                } else {
                    umma_f16(tmem_base, umma_desc(a_hi + j * 2 * kLBO, kSBO), bd, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                    if (!a.single) umma_f16(tmem_base, umma_desc(a_lo + j * 2 * kLBO, kSBO), bd, idesc, 1u);
                }
            }
            if constexpr (PAIR == 2) {                   // frees the stage in both CTAs when these MMAs retire
                umma_commit_pair(empty0 + s * 8);
                umma_commit_pair(cluster_addr(empty0 + s * 8, 1));
            } else {
                umma_commit(empty0 + s * 8);
            }
            SEQ_STAMP(kb, 4);
        }
        if (!ok) atomicExch(failed, 1);
        else if constexpr (PAIR == 2) {                  // accumulators complete, in both CTAs
            umma_commit_pair(accum_bar);
            umma_commit_pair(cluster_addr(accum_bar, 1));
        } else {
            umma_commit(accum_bar);
        }
    } else if (lane == 0) {
        // ================= second CTA of a pair: tell the first one when a stage here is full =================
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const int s = kb % S;
            ok = mbar_wait(full0 + s * 8, (kb / S) & 1);
            if (ok) mbar_arrive_remote(cluster_addr(pfull0 + s * 8, 0));
        }
        if (!ok) atomicExch(failed, 1);
    }

    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if constexpr (PAIR == 2) cluster_barrier();          // both CTAs have read their accumulators (or given up)
    else __syncthreads();
    if (*failed) {                                       // a wait gave up: give bulk copies still in flight time to land
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == kProdWarps) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if constexpr (PAIR == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BN) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BN) : "memory");
    }
    if (tid == 0 && *failed) atomicExch(a.error_flag, 1u);
}

// y[t][n] = affine(sum over the K splits, in split order) for the split-K launches.
template <typename F>
__global__ void __launch_bounds__(256) mm8_seq_reduce(int T, int M, int m_pad, int ksplit, const float* __restrict__ partial,
                                                      const float* __restrict__ sums, int nsum, const F* __restrict__ mx,
                                                      const F* __restrict__ rx, F* y, long long y_stride, const SeqEpi epi) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int t = blockIdx.y;
    float sx = 0.f, sxr = 0.f, sxmy = 0.f;
    for (int z = 0; z < nsum; ++z) {
        const float* sp = sums + ((size_t)z * T + t) * 4;
        sx += sp[0]; sxr += sp[1]; sxmy += sp[2];
    }
    for (int n = blockIdx.x * 256 + threadIdx.x; n < M; n += gridDim.x * 256) {
        float s = 0.f;
        for (int z = 0; z < ksplit; ++z) s += partial[((long long)z * T + t) * m_pad + n];
        const float rxn = to_f32<F>(rx[n]);
        y[(long long)t * y_stride + n] = seq_epilogue<F>(epi, t, n, fmaf(rxn, s, fmaf(rxn * 128.5f, sxr, fmaf(to_f32<F>(mx[n]), sx, sxmy))));
    }
}

int g_tc_single = 0;
int g_tc_no_pair = 0;

// K splits of a launch: 1 unless its output tiles (a few row tiles x the column tiles) leave most SMs idle.
static inline int tc_ksplit(int64_t B, int64_t N, int64_t M) {
    const int64_t tiles64 = ((M + BN - 1) / BN) * ((B + BM - 1) / BM);
    if (tiles64 > rwkv_sm_count() / 2) return 1;
    const int tiles = int(tiles64), nkb = int((N + BK - 1) / BK);
    int ks = rwkv_sm_count() / tiles;
    if (ks > 8) ks = 8;
    if (ks > nkb / 4) ks = nkb / 4;
    return ks < 2 ? 1 : ks;
}
static inline int64_t tc_mpad(int64_t M) { return (M + BN - 1) / BN * BN; }

}  // namespace

// Scratch of the tensor-core path: one error word, the row sums, the hi and lo operand tile images of x'
// (whole 128-row tiles x whole K blocks, fp16 each) and, for split-K launches, the fp32 partial sums
// [splits][B][M rounded up to 256].
constexpr int kMaxSumShares = 8;
static inline size_t tc_sums_end(int64_t B) { return (256 + size_t(kMaxSumShares) * size_t(B) * 16 + 255) / 256 * 256; }
static inline size_t tc_image_bytes(int64_t B, int64_t N) {          // one of hi, lo
    return size_t((B + BM - 1) / BM) * size_t((N + BK - 1) / BK) * kTileBytes;
}
extern "C" size_t rwkv_mm8_seq_tc_workspace_bytes(int64_t B, int64_t N, int64_t M) {
    const int ks = tc_ksplit(B, N, M);
    const size_t part = ks > 1 ? size_t(ks) * size_t(B) * size_t(tc_mpad(M)) * 4 : 0;
    return tc_sums_end(B) + 2 * tc_image_bytes(B, N) + part;
}

// Returns RWKV_ERR_UNSUPPORTED when the operands do not meet the layout the tensor-core kernel
// needs (the caller then uses the CUDA-core kernel).
int rwkv_mm8_seq_tc(int64_t B, int64_t N, int64_t M, const void* x, int64_t x_stride,
                    const uint8_t* w, int64_t w_stride, const void* mx, const void* rx,
                    const void* my, const void* ry, int dtype, void* y, int64_t y_stride, const SeqEpi& epi,
                    void* workspace, size_t workspace_bytes, void* stream) {
    RWKV_CHECK_ARG(B >= 1 && N >= 1 && M >= 1 && x && w && mx && rx && my && ry && y);
    if (dtype != RWKV_F16) return RWKV_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(w) % 8 != 0 || w_stride % 8 != 0 || M % 8 != 0) return RWKV_ERR_UNSUPPORTED;
    if (workspace == nullptr || workspace_bytes < rwkv_mm8_seq_tc_workspace_bytes(B, N, M)) return RWKV_ERR_WORKSPACE;
    RWKV_CHECK_ALIGN(workspace, 256);
    if ((B + BM - 1) / BM > 65535) return RWKV_ERR_UNSUPPORTED;
    const int nkb_all = int((N + BK - 1) / BK);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    unsigned* err = reinterpret_cast<unsigned*>(ws);
    float* sums = reinterpret_cast<float*>(ws + 256);
    uint8_t* hi = ws + tc_sums_end(B);
    uint8_t* lo = hi + tc_image_bytes(B, N);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int vec_x = (reinterpret_cast<uintptr_t>(x) % 16 == 0 && x_stride % 8 == 0) ? 1 : 0;
    const int vec_v = (reinterpret_cast<uintptr_t>(ry) % 16 == 0 && reinterpret_cast<uintptr_t>(my) % 16 == 0) ? 1 : 0;
    const int groups = int((B + 7) / 8);                                       // 8-row groups
    static int share_mul = -1;
    if (share_mul < 0) { const char* e = getenv("RWKV_B200_PREP_SHARES"); share_mul = e ? atoi(e) : 8; }
    int shares = std::min(kMaxSumShares, std::max(1, share_mul * rwkv_sm_count() / groups));
    shares = std::max(1, std::min(shares, nkb_all * 8 / 32));                  // at least one chunk per thread
    const int chunks_per = (nkb_all * 8 + shares - 1) / shares;
    shares = (nkb_all * 8 + chunks_per - 1) / chunks_per;                      // no empty share
    int rc = rwkv_launch_pdl(mm8_seq_prep<__half>, dim3((unsigned)groups, (unsigned)shares), dim3(256), 0, st, int(B), int(N),
                             nkb_all, static_cast<const __half*>(x), (long long)x_stride, static_cast<const __half*>(ry),
                             static_cast<const __half*>(my), vec_x, vec_v, chunks_per, hi, lo, sums);
    if (rc != RWKV_OK) return rc;
    TcArgs a;
    a.hi = hi; a.lo = lo; a.sums = sums; a.nsum = shares; a.w = w; a.w_stride = w_stride; a.mx = mx; a.rx = rx;
    a.y = y; a.y_stride = y_stride; a.T = int(B); a.N = int(N); a.M = int(M); a.error_flag = err;
    a.single = g_tc_single;
    a.epi = epi;
    a.vec_ok = (reinterpret_cast<uintptr_t>(y) % 16 == 0 && y_stride % 8 == 0 && reinterpret_cast<uintptr_t>(rx) % 16 == 0 &&
                reinterpret_cast<uintptr_t>(mx) % 16 == 0) ? 1 : 0;
    if (epi.aux != nullptr && (reinterpret_cast<uintptr_t>(epi.aux) % 16 != 0 || epi.aux_stride % 8 != 0)) a.vec_ok = 0;
    if (epi.aux2 != nullptr && (reinterpret_cast<uintptr_t>(epi.aux2) % 16 != 0 || epi.aux2_stride % 8 != 0)) a.vec_ok = 0;
    auto kern = mm8_seq_tc_kernel<__half, 1>;
    auto kern2 = mm8_seq_tc_kernel<__half, 2>;
    static bool configured[64] = {};         // function attributes are per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    if (dev >= 64 || !configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc) != cudaSuccess ||
            cudaFuncSetAttribute(kern2, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc2) != cudaSuccess) {
            cudaGetLastError();
            return RWKV_ERR_LAUNCH;
        }
        if (dev < 64) configured[dev] = true;
    }
    int ks = tc_ksplit(B, N, M);
    a.kb_per = (nkb_all + ks - 1) / ks;
    ks = (nkb_all + a.kb_per - 1) / a.kb_per;          // no empty split
    a.ksplit = ks;
    a.m_pad = int(tc_mpad(M));
    a.partial = reinterpret_cast<float*>(ws + tc_sums_end(B) + 2 * tc_image_bytes(B, N));
    dim3 grid((unsigned)((M + BN - 1) / BN), (unsigned)((B + BM - 1) / BM), (unsigned)ks);
    // an even number of row tiles and no K split: pairs of row tiles as clusters of two CTAs along x
    // (RWKV_B200_SEQ_PAIR=0 or rwkv_mm8_seq_set_path with bit 3 set: never).  Same sums in the same order: the results
    // are bit-identical to the one-CTA form; 3-4 % faster over a 1024- or 2048-token prompt at the 7B shape.
    static int use_pair = -1;
    if (use_pair < 0) { const char* e = getenv("RWKV_B200_SEQ_PAIR"); use_pair = (e != nullptr && e[0] == '0') ? 0 : 1; }
    if (use_pair && !g_tc_no_pair && ks == 1 && grid.y % 2 == 0) {
        static int use_pdl = -1;
        if (use_pdl < 0) { const char* e = getenv("RWKV_B200_PDL"); use_pdl = (e != nullptr && e[0] == '0') ? 0 : 1; }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid.x * 2, grid.y / 2, 1);
        cfg.blockDim = dim3(kThreadsTc);
        cfg.dynamicSmemBytes = size_t(kSmemTc2);
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = use_pdl ? 2 : 1;
        cudaError_t pe = cudaLaunchKernelEx(&cfg, kern2, a);
        if (pe == cudaSuccess) return RWKV_OK;
        if (getenv("RWKV_B200_VERBOSE")) {
            int nc = -1;
            cudaGetLastError();
            cudaError_t oe = cudaOccupancyMaxActiveClusters(&nc, kern2, &cfg);
            fprintf(stderr, "[rwkv-b200] pair launch: %s; max active clusters %d (%s); grid %u %u %u smem %d\n", cudaGetErrorString(pe), nc,
                    cudaGetErrorString(oe), cfg.gridDim.x, cfg.gridDim.y, cfg.gridDim.z, kSmemTc2);

        }
        cudaGetLastError();                            // no room for the pair form: the one-CTA form below
    }
    rc = rwkv_launch_pdl(kern, grid, dim3(kThreadsTc), size_t(kSmemTc), st, a);
    if (rc != RWKV_OK || ks == 1) return rc;
    return rwkv_launch_pdl(mm8_seq_reduce<__half>, dim3((unsigned)((M + 255) / 256), (unsigned)B), dim3(256), 0, st, int(B),
                           int(M), a.m_pad, ks, (const float*)a.partial, (const float*)sums, shares, static_cast<const __half*>(mx),
                           static_cast<const __half*>(rx), static_cast<__half*>(y), (long long)y_stride, epi);
}

// 1: one tensor-core pass with fp16(x*ry) instead of the exact hi + lo pair (about 1e-4 of the output RMS less
// accurate, half the tensor work); 0 (default): exact.  Set through rwkv_mm8_seq_set_path.
extern "C" void rwkv_mm8_seq_tc_set_single(int single) { g_tc_single = single ? 1 : 0; }
// 1: never the CTA-pair form of the tensor-core kernel (set through rwkv_mm8_seq_set_path, bit 3)
void rwkv_mm8_seq_tc_set_no_pair(int no_pair) { g_tc_no_pair = no_pair ? 1 : 0; }

extern "C" int rwkv_mm8_seq_tc_take_error(void* workspace, void* stream, int* error_out) {
    RWKV_CHECK_ARG(workspace != nullptr && error_out != nullptr);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned v = 0;
    if (cudaMemcpyAsync(&v, workspace, sizeof(v), cudaMemcpyDeviceToHost, st) != cudaSuccess) return RWKV_ERR_LAUNCH;
    if (cudaStreamSynchronize(st) != cudaSuccess) return RWKV_ERR_LAUNCH;
    if (v != 0 && cudaMemsetAsync(workspace, 0, sizeof(v), st) != cudaSuccess) return RWKV_ERR_LAUNCH;
    *error_out = int(v);
    return RWKV_OK;
}
