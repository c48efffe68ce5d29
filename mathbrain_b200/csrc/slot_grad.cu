// Scatter-add of per-sample slot gradients into a vocabulary-sized table.
//
// The attention backward returns dE_k and dE_v per LISTED slot of every sample ([B, K, D]); the embedding table
// receives, per token, the sum over the samples (and over K/V and layers) that list it.  The reference gets this
// sum from autograd's backward of F.embedding(safe_unique, E_slots) (mathbrain/model.py:63-68); here one kernel
// reads each gradient row once (16-byte loads), adds the K and V rows in fp32 and issues vector reductions
// (red.global.add.v4.f32) into out[token].  HBM-bound: 2 * R * D * sizeof(dtype) bytes read per call, the table
// rows it touches stay in L2.
#include "common.cuh"

namespace mbema {

constexpr int SG_WARPS = 8;

template <int DT>
__global__ void __launch_bounds__(SG_WARPS * 32)
k_slot_grad_scatter(const void* __restrict__ dA, const void* __restrict__ dB, const int64_t* __restrict__ slots,
                    float* __restrict__ out, int64_t R, int D, int64_t V) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * SG_WARPS + (threadIdx.x >> 5);
    const int64_t stride = (int64_t)gridDim.x * SG_WARPS;
    for (int64_t r = warp0; r < R; r += stride) {
        const int64_t tok = slots[r];
        if (tok < 0 || tok >= V) continue;              // -1 = not a slot
        float* dst = out + tok * D;
        for (int c = lane * 8; c < D; c += 32 * 8) {    // 8 elements per lane per pass
            float4 a0 = ld4_dyn_f32(dA, DT, (size_t)r * D + c), a1 = ld4_dyn_f32(dA, DT, (size_t)r * D + c + 4);
            if (dB) {
                float4 b0 = ld4_dyn_f32(dB, DT, (size_t)r * D + c), b1 = ld4_dyn_f32(dB, DT, (size_t)r * D + c + 4);
                a0.x += b0.x; a0.y += b0.y; a0.z += b0.z; a0.w += b0.w;
                a1.x += b1.x; a1.y += b1.y; a1.z += b1.z; a1.w += b1.w;
            }
            atomicAdd(reinterpret_cast<float4*>(dst + c), a0);
            atomicAdd(reinterpret_cast<float4*>(dst + c + 4), a1);
        }
    }
}

}  // namespace mbema

using namespace mbema;

extern "C" int mbema_slot_grad_scatter(const void* dE_a, const void* dE_b, int dtype, const int64_t* slots, float* out,
                                       int64_t R, int64_t D, int64_t V, void* stream) {
    if (R < 0 || D <= 0 || V <= 0 || D % 8 != 0 || D > (1 << 20)) return MBEMA_ERR_SHAPE;
    if (R == 0) return MBEMA_OK;
    if (!dE_a || !slots || !out) return MBEMA_ERR_NULL;
    if (dtype != MBEMA_F32 && dtype != MBEMA_BF16) return MBEMA_ERR_DTYPE;
    if (((uintptr_t)dE_a | (uintptr_t)dE_b | (uintptr_t)out) & 15) return MBEMA_ERR_ALIGN;
    int dev = 0, sms = 148;
    MBEMA_CUDA_TRY(cudaGetDevice(&dev));
    MBEMA_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t want = (R + SG_WARPS - 1) / SG_WARPS, cap = (int64_t)sms * 8;       // 8 CTAs of 8 warps per SM
    const int grid = (int)(want < cap ? want : cap);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == MBEMA_F32)
        k_slot_grad_scatter<MBEMA_F32><<<grid, SG_WARPS * 32, 0, st>>>(dE_a, dE_b, slots, out, R, (int)D, V);
    else
        k_slot_grad_scatter<MBEMA_BF16><<<grid, SG_WARPS * 32, 0, st>>>(dE_a, dE_b, slots, out, R, (int)D, V);
    return check_launch();
}

// ------------------------------------------------------------------------------------------------
// Chunk-start state of listed slots from resident per-document state:
//   c_base[b, k, :] = state[b, v, :] * rho^(t0[b] - last_t[b, v])  for v = slots[b, k] seen before, else 0.
// This is the quantity the reference's dataset computes per chunk in Python (mathbrain/data.py:128-140) from
// states.bin; with the state resident (the decode layout: value after the last update + step of that update) it is
// one gather + decay pass.  One warp per (b, k) row, channels on the lanes (coalesced 4N-byte rows).
// ------------------------------------------------------------------------------------------------
namespace mbema {

__global__ void __launch_bounds__(SG_WARPS * 32)
k_slot_state_gather(const float* __restrict__ state, const int32_t* __restrict__ last_t, const int64_t* __restrict__ slots,
                    const int32_t* __restrict__ t0, const float* __restrict__ rhos, float* __restrict__ c_base,
                    int64_t B, int64_t K, int64_t V, int N) {
    const int lane = threadIdx.x & 31;
    const int64_t R = B * K, stride = (int64_t)gridDim.x * SG_WARPS;
    for (int64_t r = (int64_t)blockIdx.x * SG_WARPS + (threadIdx.x >> 5); r < R; r += stride) {
        const int64_t b = r / K, v = slots[r];
        int lt = -1;
        if (v >= 0 && v < V) lt = last_t[b * V + v];
        const float dt = (float)(t0[b] - lt);
        for (int n = lane; n < N; n += 32) {
            float out = 0.f;
            if (lt >= 0) out = state[(b * V + v) * N + n] * exp2f(dt * log2f(rhos[n]));
            c_base[r * N + n] = out;
        }
    }
}

}  // namespace mbema

extern "C" int mbema_slot_state_gather(const float* state, const int32_t* last_t, const int64_t* slots, const int32_t* t0,
                                       const float* rhos, float* c_base, int64_t B, int64_t K, int64_t V, int64_t N,
                                       void* stream) {
    if (B < 0 || K < 0 || V <= 0 || N <= 0 || N > 1024) return MBEMA_ERR_SHAPE;
    if (B == 0 || K == 0) return MBEMA_OK;
    if (!state || !last_t || !slots || !t0 || !rhos || !c_base) return MBEMA_ERR_NULL;
    int dev = 0, sms = 148;
    MBEMA_CUDA_TRY(cudaGetDevice(&dev));
    MBEMA_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t want = (B * K + SG_WARPS - 1) / SG_WARPS, cap = (int64_t)sms * 8;
    k_slot_state_gather<<<(int)(want < cap ? want : cap), SG_WARPS * 32, 0, (cudaStream_t)stream>>>(
        state, last_t, slots, t0, rhos, c_base, B, K, V, (int)N);
    return check_launch();
}
