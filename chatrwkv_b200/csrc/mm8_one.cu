// mm8_one: decode-time dequantising GEMV, y[M] = x[N] @ dequant(W[N,M]).  HBM-bound: the
// only large operand is the uint8 matrix, read exactly once with 128-bit loads.
//
// Algebra (from the per-element form in the reference, pkg/cuda/operators.cu:224-228):
//   y[k] = rx[k] * sum_j (x[j]*ry[j]) * (w[j,k] - 128)            <- the streamed part
//        + rx[k] * 128.5 * sum_j x[j]*ry[j] + mx[k] * sum_j x[j] + sum_j x[j]*my[j]
// The byte codes are centred (w - 128) so the streamed sum does not cancel against the
// three scalar sums when x is one-signed (the FFN value matmul sees relu(k)^2 >= 0).
//
// Work split: grid = (column panels of 512, K-splits, problems).  A CTA of 8 warps owns
// 512 columns x one contiguous slice of rows; lane l of every warp owns the 16 columns
// [16 l, 16 l + 16) of the panel (one uint4 per row), warp w takes rows w, w+8, ...
// Partial sums go through shared memory (8 warps -> 1) and then through a global scratch
// buffer [split][column]; the last CTA to finish a panel (atomic ticket) adds the splits in
// split order, so the result does not depend on scheduling, and applies the epilogue.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kPanel = 512;          // columns per CTA
constexpr int kMaxRowsPerCta = 2048; // x' slice kept in shared memory
constexpr int kMaxSplit = 64;
constexpr int kCounterBytes = 4096;  // 1024 panel tickets
constexpr int kSumsBytes = (kCounterBytes / 4) * kMaxSplit * 4 * sizeof(float);  // [panel ticket][split][4]
constexpr int kMaxProblems = 3;

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
    int rows_per_cta;   // multiple of 8
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
__device__ __forceinline__ float code(uint32_t word, int i) {
    uint32_t bits = __byte_perm(word, 0x4B000000u, 0x7650 | i);
    return __uint_as_float(bits) - 8388736.0f;
}

template <bool ALIGNED>
__device__ __forceinline__ uint4 load16(const uint8_t* p, int valid) {
    if (ALIGNED) {
        uint4 v;
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
        return v;
    } else {
        uint32_t r[4] = {0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (i < valid) r[i >> 2] |= uint32_t(p[i]) << (8 * (i & 3));
        return make_uint4(r[0], r[1], r[2], r[3]);
    }
}

__device__ __forceinline__ void fma16(float (&acc)[16], const uint4& v, float xv) {
    const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[q * 4 + i] = fmaf(xv, code(wd[q], i), acc[q * 4 + i]);
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

template <typename F, bool ALIGNED>
__global__ void __launch_bounds__(kThreads, 2) mm8_one_kernel(const __grid_constant__ Batch b) {
    const Problem& P = b.p[blockIdx.z];
    const int panel = blockIdx.x;
    const int col0 = panel * kPanel;
    const int split = blockIdx.y;
    if (col0 >= P.M || split >= P.splits) return;

    __shared__ float xs[kMaxRowsPerCta];
    __shared__ float red[kWarps][kPanel];
    __shared__ float ssum[kWarps][3];
    __shared__ unsigned s_ticket;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j0 = split * P.rows_per_cta;
    const int j1 = min(P.N, j0 + P.rows_per_cta);
    const F* x = static_cast<const F*>(P.x);
    const F* ry = static_cast<const F*>(P.ry);
    const F* my = static_cast<const F*>(P.my);

    // x' = x * ry for this CTA's rows, plus this slice's share of the three scalar sums.
    float sx = 0.f, sxr = 0.f, sxmy = 0.f;
    for (int j = j0 + tid; j < j1; j += kThreads) {
        float xv = to_f32<F>(x[j]);
        float xp = xv * to_f32<F>(ry[j]);
        xs[j - j0] = xp;
        sx += xv;
        sxr += xp;
        sxmy = fmaf(xv, to_f32<F>(my[j]), sxmy);
    }
    sx = warp_sum(sx); sxr = warp_sum(sxr); sxmy = warp_sum(sxmy);
    if (lane == 0) { ssum[warp][0] = sx; ssum[warp][1] = sxr; ssum[warp][2] = sxmy; }
    __syncthreads();

    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;

    const int c = col0 + lane * 16;
    const int valid = min(16, P.M - c);         // <= 0: this lane is past the last column
    if (valid > 0) {
        const int nrows = j1 - j0;
        const uint8_t* wp = P.w + (long long)(j0 + warp) * P.w_stride + c;
        const long long step = (long long)kWarps * P.w_stride;
        constexpr int U = 8;
        int r = warp;
        for (; r + (U - 1) * kWarps < nrows; r += U * kWarps) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = load16<ALIGNED>(wp + u * step, valid);
            wp += U * step;
#pragma unroll
            for (int u = 0; u < U; ++u) fma16(acc, v[u], xs[r + u * kWarps]);
        }
        for (; r < nrows; r += kWarps) {
            uint4 v = load16<ALIGNED>(wp, valid);
            wp += step;
            fma16(acc, v, xs[r]);
        }
    }

    // 8 warps -> 1.  Element (lane, i) sits at position i*32 + lane so that both the
    // stores here and the loads below are bank-conflict free; position p holds column
    // (p % 32) * 16 + p / 32 of the panel.
#pragma unroll
    for (int i = 0; i < 16; ++i) red[warp][i * 32 + lane] = acc[i];
    __syncthreads();
    float* part = b.partial + P.partial_off + (long long)split * P.m_pad + col0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int p = tid + h * kThreads;
        float s = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < kWarps; ++w8) s += red[w8][p];
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

    // Ticket: the last CTA of this panel reduces over the splits.
    __threadfence();
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(&b.counters[P.counter_off + panel], 1u);
    __syncthreads();
    if (s_ticket != unsigned(P.splits - 1)) return;
    __threadfence();
    if (tid == 0) b.counters[P.counter_off + panel] = 0u;   // ready for the next call

    float tx = 0.f, txr = 0.f, txmy = 0.f;
    for (int sp = 0; sp < P.splits; ++sp) {
        tx += __ldcg(sums + sp * 4 + 0);
        txr += __ldcg(sums + sp * 4 + 1);
        txmy += __ldcg(sums + sp * 4 + 2);
    }

    const F* mx = static_cast<const F*>(P.mx);
    const F* rx = static_cast<const F*>(P.rx);
    const float* pbase = b.partial + P.partial_off + col0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int p = tid + h * kThreads;
        const int k = col0 + (p & 31) * 16 + (p >> 5);
        float s = 0.f;
        for (int sp = 0; sp < P.splits; ++sp) s += __ldcg(pbase + (long long)sp * P.m_pad + p);
        if (k < P.M) {
            const float rxk = to_f32<F>(rx[k]);
            const float val = fmaf(rxk, s, fmaf(rxk * 128.5f, txr, fmaf(to_f32<F>(mx[k]), tx, txmy)));
            store_epilogue<F>(P, k, val);
        }
    }
}

}  // namespace

extern "C" size_t rwkv_mm8_one_workspace_bytes(int64_t N, int64_t M) {
    (void)N;
    int64_t m_pad = (M + kPanel - 1) / kPanel * kPanel;
    return size_t(kCounterBytes) + size_t(kSumsBytes) + size_t(kMaxSplit) * size_t(m_pad) * sizeof(float);
}

extern "C" size_t rwkv_mm8_one_batch_workspace_bytes(const rwkv_mm8_problem* problems, int count) {
    size_t bytes = size_t(kCounterBytes) + size_t(kSumsBytes);
    for (int i = 0; i < count; ++i) {
        int64_t m_pad = (int64_t(problems[i].M) + kPanel - 1) / kPanel * kPanel;
        bytes += size_t(kMaxSplit) * size_t(m_pad) * sizeof(float);
    }
    return bytes;
}

static int g_split_override = 0;
extern "C" void rwkv_mm8_one_set_split(int split) { g_split_override = split; }

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

    // Total panels decide how many K-splits fill the machine about twice over.
    int total_panels = 0;
    for (int i = 0; i < count; ++i) {
        const rwkv_mm8_problem& q = problems[i];
        RWKV_CHECK_ARG(q.N >= 1 && q.M >= 1 && q.w_stride >= q.M);
        RWKV_CHECK_ARG(q.x && q.w && q.mx && q.rx && q.my && q.ry && q.y);
        RWKV_CHECK_ARG(q.epilogue >= RWKV_EPI_ACC_F32 && q.epilogue <= RWKV_EPI_STORE_F32);
        if (q.epilogue == RWKV_EPI_RESIDUAL || q.epilogue == RWKV_EPI_MUL_RESIDUAL) RWKV_CHECK_ARG(q.aux != nullptr);
        if (q.epilogue == RWKV_EPI_MUL_RESIDUAL) RWKV_CHECK_ARG(q.aux2 != nullptr);
        total_panels += (q.M + kPanel - 1) / kPanel;
    }
    if (total_panels > kCounterBytes / 4) return RWKV_ERR_UNSUPPORTED;
    const int sms = rwkv_sm_count();
    bool aligned = true;
    int max_panels = 0, max_splits = 0, counter_off = 0;
    long long partial_off = 0;
    for (int i = 0; i < count; ++i) {
        const rwkv_mm8_problem& q = problems[i];
        Problem& P = b.p[i];
        P.x = q.x; P.w = q.w; P.w_stride = q.w_stride; P.mx = q.mx; P.rx = q.rx; P.my = q.my; P.ry = q.ry;
        P.y = q.y; P.aux = q.aux; P.aux2 = q.aux2; P.N = q.N; P.M = q.M; P.epilogue = q.epilogue;
        P.out_scale = q.out_scale;
        const int panels = (q.M + kPanel - 1) / kPanel;
        // ~2 CTAs per SM over all problems, rows per CTA a multiple of 8, at least 32 rows.
        int want = g_split_override > 0 ? g_split_override : (2 * sms + total_panels - 1) / total_panels;
        int min_split = (q.N + kMaxRowsPerCta - 1) / kMaxRowsPerCta;
        int max_split = (q.N + 31) / 32;
        if (max_split > kMaxSplit) max_split = kMaxSplit;
        if (want > max_split) want = max_split;
        if (want < min_split) want = min_split;
        if (want > kMaxSplit) return RWKV_ERR_UNSUPPORTED;   // N beyond 64 * 2048 rows
        int rows = ((q.N + want - 1) / want + 7) / 8 * 8;
        P.rows_per_cta = rows;
        P.splits = (q.N + rows - 1) / rows;
        P.m_pad = panels * kPanel;
        P.partial_off = partial_off;
        P.counter_off = counter_off;
        partial_off += (long long)kMaxSplit * P.m_pad;
        counter_off += panels;
        if (panels > max_panels) max_panels = panels;
        if (P.splits > max_splits) max_splits = P.splits;
        const bool rows_padded = (q.M % 16 == 0) || (q.w_stride >= (q.M + 15) / 16 * 16);
        if (reinterpret_cast<uintptr_t>(q.w) % 16 != 0 || q.w_stride % 16 != 0 || !rows_padded) aligned = false;
    }
    for (int i = count; i < kMaxProblems; ++i) b.p[i] = b.p[0];

    dim3 grid(max_panels, max_splits, count);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == RWKV_F16) {
        if (aligned) mm8_one_kernel<__half, true><<<grid, kThreads, 0, st>>>(b);
        else mm8_one_kernel<__half, false><<<grid, kThreads, 0, st>>>(b);
    } else {
        if (aligned) mm8_one_kernel<float, true><<<grid, kThreads, 0, st>>>(b);
        else mm8_one_kernel<float, false><<<grid, kThreads, 0, st>>>(b);
    }
    return rwkv_launch_status();
}

extern "C" int rwkv_mm8_one(int64_t N, int64_t M, const void* x, const uint8_t* w, int64_t w_stride,
                            const void* mx, const void* rx, const void* my, const void* ry, int dtype,
                            float* y, void* workspace, size_t workspace_bytes, void* stream) {
    RWKV_CHECK_ARG(N >= 1 && M >= 1 && N <= INT32_MAX && M <= INT32_MAX);
    rwkv_mm8_problem q;
    q.x = x; q.w = w; q.w_stride = w_stride; q.mx = mx; q.rx = rx; q.my = my; q.ry = ry;
    q.y = y; q.aux = nullptr; q.aux2 = nullptr; q.N = int32_t(N); q.M = int32_t(M);
    q.epilogue = RWKV_EPI_ACC_F32; q.out_scale = 1.0f;
    return rwkv_mm8_one_batch(&q, 1, dtype, workspace, workspace_bytes, stream);
}
