// quantize_weight: the int8 packing of the loader (reference: pkg/model.py:818-847) as a
// sequence of min/max reductions and one coding pass, all in IEEE fp32 (explicit
// __fsub_rn / __fdiv_rn: no fast-math division, no FMA contraction), so that the codes and
// the four scale vectors are bit-identical to what the reference's CPU tensor ops produce.
//
// The source matrix is addressed through two element strides, so the loader's transposed
// view of an [out, in] nn.Linear weight is packed without a transposing copy.  Reductions
// along the contiguous source axis use one warp per line; reductions along the strided axis
// use one thread per column and chunks of 512 lines, combined by a second small kernel
// (min and max do not depend on the order of combination).
#include "common.cuh"

namespace {

struct QArgs {
    const void* src;
    long long sn, sm;     // element strides of the reduction index j and the output index k
    float scale;
    int N, M;
    int row_first;        // N > M: subtract the row minimum (my) first
    int c_is_k;           // the contiguous source axis is k
    float *mx, *rx, *my, *ry;   // fp32 working copies
};

template <typename S>
__device__ __forceinline__ float load_w(const QArgs& a, int j, int k) {
    const S* p = static_cast<const S*>(a.src);
    // The reference divides by 2^n in the checkpoint dtype before widening.
    return to_f32<S>(from_f32<S>(to_f32<S>(p[(long long)j * a.sn + (long long)k * a.sm]) * a.scale));
}

// STAGE 0: W   1: W - first min   2: ... - second min   3: ... / rx[k]   4: ... / ry[j]
template <typename S, int STAGE>
__device__ __forceinline__ float stage_value(const QArgs& a, int j, int k) {
    float v = load_w<S>(a, j, k);
    if (STAGE >= 1) v = __fsub_rn(v, a.row_first ? a.my[j] : a.mx[k]);
    if (STAGE >= 2) v = __fsub_rn(v, a.row_first ? a.mx[k] : a.my[j]);
    if (STAGE >= 3) v = __fdiv_rn(v, a.rx[k]);
    if (STAGE >= 4) v = __fdiv_rn(v, a.ry[j]);
    return v;
}

constexpr int kChunk = 512;

// Reduce along the CONTIGUOUS source axis: one warp per line of the strided axis.
template <typename S, int STAGE, bool IS_MAX>
__global__ void reduce_contig(const QArgs a, float* out) {
    const int line = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int lines = a.c_is_k ? a.N : a.M;
    const int len = a.c_is_k ? a.M : a.N;
    if (line >= lines) return;
    float r = IS_MAX ? -INFINITY : INFINITY;
    for (int c = lane; c < len; c += 32) {
        float v = a.c_is_k ? stage_value<S, STAGE>(a, line, c) : stage_value<S, STAGE>(a, c, line);
        r = IS_MAX ? fmaxf(r, v) : fminf(r, v);
    }
    r = IS_MAX ? warp_max(r) : warp_min(r);
    if (lane == 0) out[line] = r;
}

// Reduce along the STRIDED source axis: thread per contiguous index, chunk of lines per
// blockIdx.y; partial[chunk][c].
template <typename S, int STAGE, bool IS_MAX>
__global__ void reduce_strided(const QArgs a, float* partial) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int len = a.c_is_k ? a.M : a.N;      // extent of the contiguous axis
    const int lines = a.c_is_k ? a.N : a.M;
    if (c >= len) return;
    const int l0 = blockIdx.y * kChunk, l1 = min(lines, l0 + kChunk);
    float r = IS_MAX ? -INFINITY : INFINITY;
#pragma unroll 4
    for (int l = l0; l < l1; ++l) {
        float v = a.c_is_k ? stage_value<S, STAGE>(a, l, c) : stage_value<S, STAGE>(a, c, l);
        r = IS_MAX ? fmaxf(r, v) : fminf(r, v);
    }
    partial[(long long)blockIdx.y * len + c] = r;
}

template <bool IS_MAX>
__global__ void combine_chunks(const float* partial, int chunks, int len, float* out) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= len) return;
    float r = IS_MAX ? -INFINITY : INFINITY;
    for (int i = 0; i < chunks; ++i) {
        float v = partial[(long long)i * len + c];
        r = IS_MAX ? fmaxf(r, v) : fminf(r, v);
    }
    out[c] = r;
}

__device__ __forceinline__ uint8_t encode(float v) {
    // clip(floor(v * 256), 0, 255).to(uint8)   (pkg/model.py:843)
    float f = floorf(__fmul_rn(v, 256.0f));
    f = fminf(fmaxf(f, 0.0f), 255.0f);
    return (uint8_t)(int)f;
}

// Coding pass; 32x32 tiles so that both the source read and the q write are coalesced
// whichever source axis is contiguous.
template <typename S>
__global__ void code_pass(const QArgs a, uint8_t* q, long long q_stride) {
    __shared__ uint8_t tile[32][33];
    const int k0 = blockIdx.x * 32, j0 = blockIdx.y * 32;
    const int tx = threadIdx.x, ty = threadIdx.y;   // 32 x 8
    if (a.c_is_k) {
        for (int r = ty; r < 32; r += 8) {
            int j = j0 + r, k = k0 + tx;
            if (j < a.N && k < a.M) q[(long long)j * q_stride + k] = encode(stage_value<S, 4>(a, j, k));
        }
    } else {
        for (int r = ty; r < 32; r += 8) {
            int k = k0 + r, j = j0 + tx;
            if (j < a.N && k < a.M) tile[tx][r] = encode(stage_value<S, 4>(a, j, k));
        }
        __syncthreads();
        for (int r = ty; r < 32; r += 8) {
            int j = j0 + r, k = k0 + tx;
            if (j < a.N && k < a.M) q[(long long)j * q_stride + k] = tile[r][tx];
        }
    }
}

template <typename F>
__global__ void finalize_scales(const QArgs a, F* mx, F* rx, F* my, F* ry) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < a.M) {
        mx[i] = from_f32<F>(a.mx[i]);
        rx[i] = from_f32<F>(__fdiv_rn(a.rx[i], 16.0f));
    }
    if (i < a.N) {
        my[i] = from_f32<F>(a.my[i]);
        ry[i] = from_f32<F>(__fdiv_rn(a.ry[i], 16.0f));
    }
}

// out[j] (over_k = true) or out[k] (over_k = false) = min/max of STAGE over the other index
template <typename S, int STAGE, bool IS_MAX>
void reduce(const QArgs& a, bool over_k, float* out, float* partial, cudaStream_t st) {
    const bool along_contig = (over_k == (a.c_is_k != 0));
    if (along_contig) {
        const int lines = a.c_is_k ? a.N : a.M;
        reduce_contig<S, STAGE, IS_MAX><<<(lines + 7) / 8, 256, 0, st>>>(a, out);
    } else {
        const int len = a.c_is_k ? a.M : a.N;
        const int lines = a.c_is_k ? a.N : a.M;
        const int chunks = (lines + kChunk - 1) / kChunk;
        dim3 grid((len + 127) / 128, chunks);
        reduce_strided<S, STAGE, IS_MAX><<<grid, 128, 0, st>>>(a, partial);
        combine_chunks<IS_MAX><<<(len + 255) / 256, 256, 0, st>>>(partial, chunks, len, out);
    }
}

template <typename S>
int run(QArgs a, uint8_t* q, long long q_stride, void* mx, void* rx, void* my, void* ry,
        int scale_dtype, float* partial, cudaStream_t st) {
    if (a.row_first) {
        reduce<S, 0, false>(a, true, a.my, partial, st);
        reduce<S, 1, false>(a, false, a.mx, partial, st);
    } else {
        reduce<S, 0, false>(a, false, a.mx, partial, st);
        reduce<S, 1, false>(a, true, a.my, partial, st);
    }
    reduce<S, 2, true>(a, false, a.rx, partial, st);
    reduce<S, 3, true>(a, true, a.ry, partial, st);
    dim3 grid((a.M + 31) / 32, (a.N + 31) / 32);
    code_pass<S><<<grid, dim3(32, 8), 0, st>>>(a, q, q_stride);
    const int n = a.N > a.M ? a.N : a.M;
    if (scale_dtype == RWKV_F16)
        finalize_scales<__half><<<(n + 255) / 256, 256, 0, st>>>(a, (__half*)mx, (__half*)rx, (__half*)my, (__half*)ry);
    else
        finalize_scales<float><<<(n + 255) / 256, 256, 0, st>>>(a, (float*)mx, (float*)rx, (float*)my, (float*)ry);
    return rwkv_launch_status();
}

}  // namespace

extern "C" size_t rwkv_quantize_weight_workspace_bytes(int64_t N, int64_t M) {
    if (N < 1 || M < 1) return 0;
    const int64_t big = N > M ? N : M;
    const int64_t chunks = (big + kChunk - 1) / kChunk;
    return size_t(2 * (N + M) + chunks * big) * sizeof(float);
}

extern "C" int rwkv_quantize_weight(const void* src, int src_dtype, int64_t src_stride_n, int64_t src_stride_m,
                                    float scale, int64_t N, int64_t M, uint8_t* q, int64_t q_stride,
                                    void* mx, void* rx, void* my, void* ry, int scale_dtype,
                                    void* workspace, size_t workspace_bytes, void* stream) {
    RWKV_CHECK_ARG(src && q && mx && rx && my && ry);
    RWKV_CHECK_ARG(N >= 1 && M >= 1 && N <= INT32_MAX && M <= INT32_MAX && q_stride >= M);
    RWKV_CHECK_ARG(src_stride_n >= 1 && src_stride_m >= 1);
    RWKV_CHECK_ARG(scale_dtype == RWKV_F16 || scale_dtype == RWKV_F32);
    RWKV_CHECK_ARG((M + 31) / 32 <= 0x7fffffff && (N + 31) / 32 <= 65535 * 32);
    if (workspace == nullptr || workspace_bytes < rwkv_quantize_weight_workspace_bytes(N, M)) return RWKV_ERR_WORKSPACE;
    RWKV_CHECK_ALIGN(workspace, 16);
    QArgs a;
    a.src = src; a.sn = src_stride_n; a.sm = src_stride_m; a.scale = scale;
    a.N = int(N); a.M = int(M);
    a.row_first = N > M;                       // pkg/model.py:824
    a.c_is_k = src_stride_m <= src_stride_n;
    float* ws = static_cast<float*>(workspace);
    a.mx = ws; a.rx = ws + M; a.my = ws + 2 * M; a.ry = ws + 2 * M + N;
    float* partial = ws + 2 * (M + N);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if ((N + 31) / 32 > 65535) return RWKV_ERR_UNSUPPORTED;
    switch (src_dtype) {
    case RWKV_F32: return run<float>(a, q, q_stride, mx, rx, my, ry, scale_dtype, partial, st);
    case RWKV_F16: return run<__half>(a, q, q_stride, mx, rx, my, ry, scale_dtype, partial, st);
    case RWKV_BF16: return run<__nv_bfloat16>(a, q, q_stride, mx, rx, my, ry, scale_dtype, partial, st);
    default: return RWKV_ERR_INVALID_ARG;
    }
}
