// Gather + LayerNorm over the DISTINCT tokens listed in a batch: memory_base[u, :] = LN(E[tokens[u], :]).
//
// The reference gathers and normalises per sample and layer (mathbrain/model.py:63-65: F.embedding(safe_unique,
// E_slots) then ln_kv over [B, K_max, D]); most listed tokens recur across the samples of a batch, so the rows are
// normalised (and then projected by the caller's k_proj / v_proj GEMMs) once per distinct token instead.  The
// backward fuses the LayerNorm backward with the scatter into the embedding gradient: dE[tokens[u], :] += dx.
// HBM-bound: forward reads U*D table elements and writes U*D; backward reads 2*U*D and adds U*D (fp32 vector
// reductions; the tokens of one call are distinct, the adds only serialise against other layers' calls).
#include "common.cuh"

namespace mbema {

constexpr int SLN_WARPS = 8;
constexpr int SLN_MAXV = 8;          // float4 chunks per lane: D <= 32 * 4 * 8 = 1024

struct SlotLnArgs {
    const void* E; int e_dt;
    const int64_t* tokens;
    const float* ln_w; const float* ln_b; float eps;
    void* out; int out_dt;           // forward
    float* mu; float* rstd;
    const void* dY; int dy_dt;       // backward
    float* dE; float* dln_w; float* dln_b;
    int64_t U; int D; int64_t V;
};

template <int NV>
__global__ void __launch_bounds__(SLN_WARPS * 32) k_slot_ln_fwd(SlotLnArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t stride = (int64_t)gridDim.x * SLN_WARPS;
    const float invD = 1.0f / (float)a.D;
    for (int64_t u = (int64_t)blockIdx.x * SLN_WARPS + (threadIdx.x >> 5); u < a.U; u += stride) {
        const int64_t tok = a.tokens[u];
        const bool ok = tok >= 0 && tok < a.V;
        float4 x[NV];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = (lane + 32 * i) * 4;
            x[i] = (ok && c < a.D) ? ld4_dyn_f32(a.E, a.e_dt, (size_t)tok * a.D + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            s += x[i].x + x[i].y + x[i].z + x[i].w;
        }
        const float mean = warp_sum(s) * invD;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = (lane + 32 * i) * 4;
            if (c < a.D) {
                const float d0 = x[i].x - mean, d1 = x[i].y - mean, d2 = x[i].z - mean, d3 = x[i].w - mean;
                q += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
            }
        }
        const float rstd = rsqrtf(warp_sum(q) * invD + a.eps);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = (lane + 32 * i) * 4;
            if (c < a.D) {
                const float4 w = *reinterpret_cast<const float4*>(a.ln_w + c), bb = *reinterpret_cast<const float4*>(a.ln_b + c);
                float4 y;
                y.x = (x[i].x - mean) * rstd * w.x + bb.x;
                y.y = (x[i].y - mean) * rstd * w.y + bb.y;
                y.z = (x[i].z - mean) * rstd * w.z + bb.z;
                y.w = (x[i].w - mean) * rstd * w.w + bb.w;
                if (!ok) y = make_float4(0.f, 0.f, 0.f, 0.f);       // not a token: a zero row
                st4_dyn(a.out, a.out_dt, (size_t)u * a.D + c, y);
            }
        }
        if (lane == 0) { a.mu[u] = mean; a.rstd[u] = rstd; }
    }
}

template <int NV>
__global__ void __launch_bounds__(SLN_WARPS * 32) k_slot_ln_bwd(SlotLnArgs a) {
    extern __shared__ float red[];                  // [SLN_WARPS][2][D]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t stride = (int64_t)gridDim.x * SLN_WARPS;
    const float invD = 1.0f / (float)a.D;
    float4 gw[NV], gb[NV];                          // this lane's columns of dln_w / dln_b over the warp's rows
#pragma unroll
    for (int i = 0; i < NV; ++i) gw[i] = gb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t u = (int64_t)blockIdx.x * SLN_WARPS + warp; u < a.U; u += stride) {
        const int64_t tok = a.tokens[u];
        if (tok < 0 || tok >= a.V) continue;        // warp-uniform
        const float mean = a.mu[u], rstd = a.rstd[u];
        float4 xh[NV], dyw[NV];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = (lane + 32 * i) * 4;
            xh[i] = dyw[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < a.D) {
                const float4 x = ld4_dyn_f32(a.E, a.e_dt, (size_t)tok * a.D + c);
                const float4 dy = ld4_dyn_f32(a.dY, a.dy_dt, (size_t)u * a.D + c);
                const float4 w = *reinterpret_cast<const float4*>(a.ln_w + c);
                xh[i] = make_float4((x.x - mean) * rstd, (x.y - mean) * rstd, (x.z - mean) * rstd, (x.w - mean) * rstd);
                dyw[i] = make_float4(dy.x * w.x, dy.y * w.y, dy.z * w.z, dy.w * w.w);
                gw[i].x += dy.x * xh[i].x; gw[i].y += dy.y * xh[i].y; gw[i].z += dy.z * xh[i].z; gw[i].w += dy.w * xh[i].w;
                gb[i].x += dy.x; gb[i].y += dy.y; gb[i].z += dy.z; gb[i].w += dy.w;
                s1 += dyw[i].x + dyw[i].y + dyw[i].z + dyw[i].w;
                s2 += dyw[i].x * xh[i].x + dyw[i].y * xh[i].y + dyw[i].z * xh[i].z + dyw[i].w * xh[i].w;
            }
        }
        s1 = warp_sum(s1) * invD;
        s2 = warp_sum(s2) * invD;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = (lane + 32 * i) * 4;
            if (c < a.D) {
                float4 dx;
                dx.x = rstd * (dyw[i].x - s1 - xh[i].x * s2);
                dx.y = rstd * (dyw[i].y - s1 - xh[i].y * s2);
                dx.z = rstd * (dyw[i].z - s1 - xh[i].z * s2);
                dx.w = rstd * (dyw[i].w - s1 - xh[i].w * s2);
                atomicAdd(reinterpret_cast<float4*>(a.dE + (size_t)tok * a.D + c), dx);
            }
        }
    }
    // column sums of the CTA's warps, then one atomic per column and CTA
    float* rw = red + (size_t)warp * 2 * a.D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (lane + 32 * i) * 4;
        if (c < a.D) {
            *reinterpret_cast<float4*>(rw + c) = gw[i];
            *reinterpret_cast<float4*>(rw + a.D + c) = gb[i];
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < 2 * a.D; c += blockDim.x) {
        float s = 0.f;
#pragma unroll
        for (int wi = 0; wi < SLN_WARPS; ++wi) s += red[(size_t)wi * 2 * a.D + c];
        atomicAdd((c < a.D ? a.dln_w + c : a.dln_b + (c - a.D)), s);
    }
}

static int sln_grid(int64_t U) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t want = (U + SLN_WARPS - 1) / SLN_WARPS, cap = (int64_t)sms * 4;
    return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}

static int sln_check(int64_t U, int64_t D, int64_t V) {
    if (U < 0 || D <= 0 || V <= 0 || D % 4 != 0 || D > 32 * 4 * SLN_MAXV) return MBEMA_ERR_SHAPE;
    return MBEMA_OK;
}

}  // namespace mbema

using namespace mbema;

#define MBEMA_SLN_DISPATCH(KERNEL, ...)                                   \
    do {                                                                  \
        if (D <= 128) KERNEL<1> __VA_ARGS__;                              \
        else if (D <= 256) KERNEL<2> __VA_ARGS__;                         \
        else if (D <= 512) KERNEL<4> __VA_ARGS__;                         \
        else KERNEL<8> __VA_ARGS__;                                       \
    } while (0)

extern "C" int mbema_slot_ln_fwd(const void* E, int e_dtype, const int64_t* tokens, const float* ln_w, const float* ln_b,
                                 float eps, void* out, int out_dtype, float* mu, float* rstd, int64_t U, int64_t D,
                                 int64_t V, void* stream) {
    int rc = sln_check(U, D, V);
    if (rc) return rc;
    if (U == 0) return MBEMA_OK;
    if (!E || !tokens || !ln_w || !ln_b || !out || !mu || !rstd) return MBEMA_ERR_NULL;
    if ((e_dtype != MBEMA_F32 && e_dtype != MBEMA_BF16) || (out_dtype != MBEMA_F32 && out_dtype != MBEMA_BF16)) return MBEMA_ERR_DTYPE;
    if (((uintptr_t)E | (uintptr_t)ln_w | (uintptr_t)ln_b | (uintptr_t)out) & 15) return MBEMA_ERR_ALIGN;
    SlotLnArgs a{E, e_dtype, tokens, ln_w, ln_b, eps, out, out_dtype, mu, rstd, nullptr, 0, nullptr, nullptr, nullptr, U, (int)D, V};
    cudaStream_t st = (cudaStream_t)stream;
    const int grid = sln_grid(U);
    MBEMA_SLN_DISPATCH(k_slot_ln_fwd, <<<grid, SLN_WARPS * 32, 0, st>>>(a));
    return check_launch();
}

extern "C" int mbema_slot_ln_bwd(const void* dY, int dy_dtype, const void* E, int e_dtype, const int64_t* tokens,
                                 const float* ln_w, const float* mu, const float* rstd, float* dE, float* dln_w,
                                 float* dln_b, int64_t U, int64_t D, int64_t V, void* stream) {
    int rc = sln_check(U, D, V);
    if (rc) return rc;
    if (U == 0) return MBEMA_OK;
    if (!dY || !E || !tokens || !ln_w || !mu || !rstd || !dE || !dln_w || !dln_b) return MBEMA_ERR_NULL;
    if ((e_dtype != MBEMA_F32 && e_dtype != MBEMA_BF16) || (dy_dtype != MBEMA_F32 && dy_dtype != MBEMA_BF16)) return MBEMA_ERR_DTYPE;
    if (((uintptr_t)E | (uintptr_t)ln_w | (uintptr_t)dY | (uintptr_t)dE) & 15) return MBEMA_ERR_ALIGN;
    SlotLnArgs a{E, e_dtype, tokens, ln_w, nullptr, 0.f, nullptr, 0, const_cast<float*>(mu), const_cast<float*>(rstd), dY, dy_dtype, dE, dln_w, dln_b, U, (int)D, V};
    cudaStream_t st = (cudaStream_t)stream;
    const int grid = sln_grid(U);
    const size_t smem = (size_t)SLN_WARPS * 2 * D * sizeof(float);      // <= 64 KB at D = 1024
    if (smem > 48 * 1024) {
        MBEMA_CUDA_TRY(cudaFuncSetAttribute(k_slot_ln_bwd<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    MBEMA_SLN_DISPATCH(k_slot_ln_bwd, <<<grid, SLN_WARPS * 32, smem, st>>>(a));
    return check_launch();
}
