// Fused epilogues of mm8_seq: what the reference's seq functions apply to a matmul's fp16 result before the
// next one (cuda_att_seq / ffn_seq, pkg/model.py:995-1004, 1346-1360), with the same roundings as the
// decode epilogues (RWKV_EPI_* in include/rwkv_b200.h): `val` is the fp32 sum, rounded once to the output
// type; every further torch op of the reference is one more rounding.
#pragma once
#include "common.cuh"

struct SeqEpi {
    int mode;                   // RWKV_EPI_STORE, _SIGMOID, _RELU_SQ, _RESIDUAL, _MUL_RESIDUAL, _SILU
    float out_scale;
    const void* aux;            // [B, M] rows aux_stride apart, the output's dtype
    long long aux_stride;
    const void* aux2;
    long long aux2_stride;
};

template <typename F> __device__ __forceinline__ float seq_round(float v) { return to_f32<F>(from_f32<F>(v)); }

// value to store at (row t, column n); auxv / aux2v already loaded (0 when the mode does not use them)
template <typename F>
__device__ __forceinline__ F seq_epilogue_with(int mode, float out_scale, float val, float auxv, float aux2v) {
    const float v = seq_round<F>(val);
    switch (mode) {
    case RWKV_EPI_SIGMOID: return from_f32<F>(1.0f / (1.0f + expf(-v)));
    case RWKV_EPI_RELU_SQ: { const float r = fmaxf(v, 0.0f); return from_f32<F>(r * r); }
    case RWKV_EPI_RESIDUAL: return from_f32<F>(seq_round<F>(auxv + v) * out_scale);
    case RWKV_EPI_MUL_RESIDUAL: return from_f32<F>(seq_round<F>(auxv + seq_round<F>(aux2v * v)) * out_scale);
    case RWKV_EPI_SILU: return from_f32<F>(v / (1.0f + expf(-v)));
    default: return from_f32<F>(val);
    }
}

template <typename F>
__device__ __forceinline__ F seq_epilogue(const SeqEpi& e, long long t, int n, float val) {
    float auxv = 0.f, aux2v = 0.f;
    if (e.mode == RWKV_EPI_RESIDUAL || e.mode == RWKV_EPI_MUL_RESIDUAL) auxv = to_f32<F>(static_cast<const F*>(e.aux)[t * e.aux_stride + n]);
    if (e.mode == RWKV_EPI_MUL_RESIDUAL) aux2v = to_f32<F>(static_cast<const F*>(e.aux2)[t * e.aux2_stride + n]);
    return seq_epilogue_with<F>(e.mode, e.out_scale, val, auxv, aux2v);
}

static inline int seq_epi_check(const SeqEpi& e) {
    if (e.mode != RWKV_EPI_STORE && e.mode != RWKV_EPI_SIGMOID && e.mode != RWKV_EPI_RELU_SQ && e.mode != RWKV_EPI_RESIDUAL &&
        e.mode != RWKV_EPI_MUL_RESIDUAL && e.mode != RWKV_EPI_SILU)
        return RWKV_ERR_INVALID_ARG;
    if ((e.mode == RWKV_EPI_RESIDUAL || e.mode == RWKV_EPI_MUL_RESIDUAL) && e.aux == nullptr) return RWKV_ERR_INVALID_ARG;
    if (e.mode == RWKV_EPI_MUL_RESIDUAL && e.aux2 == nullptr) return RWKV_ERR_INVALID_ARG;
    return RWKV_OK;
}
