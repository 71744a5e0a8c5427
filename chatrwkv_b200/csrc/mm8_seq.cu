// mm8_seq: prefill-time dequantising GEMM  y[B,M] = x[B,N] @ dequant(W[N,M]).
//
// Same factorisation as mm8_one:  y[i,k] = rx[k] * sum_j x'[i,j] (w[j,k]-128)
//                                        + rx[k]*128.5*SXR[i] + mx[k]*SX[i] + SXMY[i]
// with x' = x*ry, SX = sum_j x, SXR = sum_j x', SXMY = sum_j x*my (per row i).
//
// This file holds the shape-agnostic CUDA-core kernel (any B, N, M, any stride or
// alignment).  It is the path for ragged or misaligned operands and for small B.
#include "common.cuh"
#include "seq_epi.cuh"

namespace {

constexpr int TM = 64;   // rows of x per CTA
constexpr int TN = 64;   // columns of W per CTA
constexpr int TK = 32;   // reduction slice

template <typename F>
__global__ void __launch_bounds__(256) mm8_seq_simt(int B, int N, int M,
                                                    const F* __restrict__ x, long long x_stride,
                                                    const uint8_t* __restrict__ w, long long w_stride,
                                                    const F* __restrict__ mx, const F* __restrict__ rx,
                                                    const F* __restrict__ my, const F* __restrict__ ry,
                                                    F* y, long long y_stride, const SeqEpi epi) {
    __shared__ float xs[TK][TM + 4];
    __shared__ float ws[TK][TN];
    __shared__ float rsum[3][TM];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int i0 = blockIdx.y * TM, k0 = blockIdx.x * TN;

    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
    // Row sums: thread (row = tid / 4, quarter = tid % 4) covers 8 of the 32 j's of a slice.
    float sx = 0.f, sxr = 0.f, sxmy = 0.f;
    const int lr = tid >> 2, lq = tid & 3;

    for (int jb = 0; jb < N; jb += TK) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int jj = lq * 8 + e, j = jb + jj, i = i0 + lr;
            float xp = 0.f;
            if (i < B && j < N) {
                const float xv = to_f32<F>(x[(long long)i * x_stride + j]);
                xp = xv * to_f32<F>(ry[j]);
                sx += xv;
                sxr += xp;
                sxmy = fmaf(xv, to_f32<F>(my[j]), sxmy);
            }
            xs[jj][lr] = xp;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int idx = tid + e * 256, jj = idx >> 6, kk = idx & 63;
            const int j = jb + jj, k = k0 + kk;
            ws[jj][kk] = (j < N && k < M) ? float(int(w[(long long)j * w_stride + k]) - 128) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int jj = 0; jj < TK; ++jj) {
            const float4 xa = *reinterpret_cast<const float4*>(&xs[jj][ty * 4]);
            const float4 wb = *reinterpret_cast<const float4*>(&ws[jj][tx * 4]);
            const float xv[4] = {xa.x, xa.y, xa.z, xa.w};
            const float wv[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(xv[a], wv[b], acc[a][b]);
        }
        __syncthreads();
    }
    // combine the four quarters of each row sum
    sx += __shfl_xor_sync(0xffffffffu, sx, 1); sx += __shfl_xor_sync(0xffffffffu, sx, 2);
    sxr += __shfl_xor_sync(0xffffffffu, sxr, 1); sxr += __shfl_xor_sync(0xffffffffu, sxr, 2);
    sxmy += __shfl_xor_sync(0xffffffffu, sxmy, 1); sxmy += __shfl_xor_sync(0xffffffffu, sxmy, 2);
    if (lq == 0) { rsum[0][lr] = sx; rsum[1][lr] = sxr; rsum[2][lr] = sxmy; }
    __syncthreads();
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const int k = k0 + tx * 4 + b;
        if (k >= M) continue;
        const float rxk = to_f32<F>(rx[k]), mxk = to_f32<F>(mx[k]);
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int r = ty * 4 + a, i = i0 + r;
            if (i >= B) continue;
            const float val = fmaf(rxk, acc[a][b], fmaf(rxk * 128.5f, rsum[1][r], fmaf(mxk, rsum[0][r], rsum[2][r])));
            y[(long long)i * y_stride + k] = seq_epilogue<F>(epi, i, k, val);
        }
    }
}

}  // namespace

// tensor-core path (mm8_seq_tc.cu)
extern "C" size_t rwkv_mm8_seq_tc_workspace_bytes(int64_t B, int64_t N, int64_t M);
int rwkv_mm8_seq_tc(int64_t B, int64_t N, int64_t M, const void* x, int64_t x_stride,
                    const uint8_t* w, int64_t w_stride, const void* mx, const void* rx,
                    const void* my, const void* ry, int dtype, void* y, int64_t y_stride, const SeqEpi& epi,
                    void* workspace, size_t workspace_bytes, void* stream);

extern "C" void rwkv_mm8_seq_tc_set_single(int single);
void rwkv_mm8_seq_tc_set_no_pair(int no_pair);
static int g_seq_path = 0;      // 0 = automatic, 1 = CUDA cores only, 2 = tensor cores whenever the layout allows
// bit 2 (value 4) of `path`: the tensor-core kernel multiplies fp16(x*ry) in one pass instead of the exact
// hi + lo pair; bit 3 (value 8): one CTA per output tile always (never the CTA-pair form; same results)
extern "C" void rwkv_mm8_seq_set_path(int path) {
    g_seq_path = path & 3;
    rwkv_mm8_seq_tc_set_single((path & 4) != 0);
    rwkv_mm8_seq_tc_set_no_pair((path & 8) != 0);
}
constexpr int kTcMinRows = 8;   // below this the CUDA-core kernel; from here on the 128-row tensor-core tile (mostly padding up to
                                // 64 rows, but 4x faster than the CUDA-core kernel already at 16 rows: W is converted once per CTA)

extern "C" size_t rwkv_mm8_seq_workspace_bytes(int64_t B, int64_t N, int64_t M) {
    if (B < 1 || N < 1 || M < 1) return 0;
    return rwkv_mm8_seq_tc_workspace_bytes(B, N, M);
}

extern "C" int rwkv_mm8_seq_epi(int64_t B, int64_t N, int64_t M, const void* x, int64_t x_stride,
                                const uint8_t* w, int64_t w_stride,
                                const void* mx, const void* rx, const void* my, const void* ry, int dtype,
                                void* y, int64_t y_stride, int epilogue, const void* aux, int64_t aux_stride,
                                const void* aux2, int64_t aux2_stride, float out_scale,
                                void* workspace, size_t workspace_bytes, void* stream) {
    RWKV_CHECK_ARG(B >= 1 && N >= 1 && M >= 1 && N <= INT32_MAX && M <= INT32_MAX && B <= INT32_MAX);
    RWKV_CHECK_ARG(x && w && mx && rx && my && ry && y);
    RWKV_CHECK_ARG(x_stride >= N && w_stride >= M && y_stride >= M);
    RWKV_CHECK_ARG(dtype == RWKV_F16 || dtype == RWKV_F32);
    SeqEpi epi;
    epi.mode = epilogue; epi.out_scale = out_scale; epi.aux = aux; epi.aux_stride = aux_stride; epi.aux2 = aux2; epi.aux2_stride = aux2_stride;
    const int erc = seq_epi_check(epi);
    if (erc != RWKV_OK) return erc;
    if (g_seq_path != 1 && workspace != nullptr && (B >= kTcMinRows || g_seq_path == 2)) {
        const int rc = rwkv_mm8_seq_tc(B, N, M, x, x_stride, w, w_stride, mx, rx, my, ry, dtype, y, y_stride, epi,
                                       workspace, workspace_bytes, stream);
        if (rc != RWKV_ERR_UNSUPPORTED && rc != RWKV_ERR_WORKSPACE) return rc;   // else: CUDA-core kernel below
    }
    dim3 grid((unsigned)((M + TN - 1) / TN), (unsigned)((B + TM - 1) / TM));
    if (grid.y > 65535) return RWKV_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == RWKV_F16)
        mm8_seq_simt<__half><<<grid, 256, 0, st>>>(int(B), int(N), int(M), (const __half*)x, x_stride, w, w_stride,
                                                    (const __half*)mx, (const __half*)rx, (const __half*)my,
                                                    (const __half*)ry, (__half*)y, y_stride, epi);
    else
        mm8_seq_simt<float><<<grid, 256, 0, st>>>(int(B), int(N), int(M), (const float*)x, x_stride, w, w_stride,
                                                   (const float*)mx, (const float*)rx, (const float*)my,
                                                   (const float*)ry, (float*)y, y_stride, epi);
    return rwkv_launch_status();
}

extern "C" int rwkv_mm8_seq(int64_t B, int64_t N, int64_t M, const void* x, int64_t x_stride,
                            const uint8_t* w, int64_t w_stride,
                            const void* mx, const void* rx, const void* my, const void* ry, int dtype,
                            void* y, int64_t y_stride, void* workspace, size_t workspace_bytes, void* stream) {
    return rwkv_mm8_seq_epi(B, N, M, x, x_stride, w, w_stride, mx, rx, my, ry, dtype, y, y_stride, RWKV_EPI_STORE, nullptr, 0,
                            nullptr, 0, 1.0f, workspace, workspace_bytes, stream);
}
