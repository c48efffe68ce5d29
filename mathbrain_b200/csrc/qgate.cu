// Query gate + LayerNorm:  Y = LN(x_q * gate(p_pre + bias)) * ln_w + ln_b   (forward and backward).
//
// HBM-bound elementwise/row-reduction work: one warp per row, 16-byte vector loads, the whole row kept in
// registers (D <= 1024), so every input is read once and every output written once.  The backward
// recomputes the gate instead of re-reading saved activations (the reference saves x_emb and p_gate,
// mathbrain/triton_fused_gating.py:142-147) and reduces the per-column sums (dbias, dln_w, dln_b) in two
// deterministic stages: per-CTA partials in the workspace, then one column-sum kernel.
#include "common.cuh"

namespace mbema {

static constexpr int QG_WARPS = 8;
// NV = float4 slots per lane (template parameter): D <= 128 * NV, NV in {1, 2, 4, 8} -> D <= 1024

struct QGateFwdArgs {
    const void* x; int x_dt;
    const void* p; int p_dt;
    const float* bias; const float* ln_w; const float* ln_b;
    float eps;
    void* y; int y_dt;
    float* mu; float* rstd;
    long long rows; int D; int silu;
};

template <int NV>
__global__ void __launch_bounds__(QG_WARPS * 32, NV <= 4 ? 4 : 2) k_qgate_fwd(QGateFwdArgs a) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    constexpr int nv = NV;
    const float invD = 1.0f / (float)a.D;
    for (long long row = (long long)blockIdx.x * QG_WARPS + warp; row < a.rows; row += (long long)gridDim.x * QG_WARPS) {
        float4 e[NV];
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = (i * 32 + lane) * 4;
            e[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < nv && d < a.D) {
                float4 xv = ld4_dyn_f32(a.x, a.x_dt, (size_t)row * a.D + d);
                float4 pv = ld4_dyn_f32(a.p, a.p_dt, (size_t)row * a.D + d);
                float4 bv = *reinterpret_cast<const float4*>(a.bias + d);
                float pl[4] = {pv.x + bv.x, pv.y + bv.y, pv.z + bv.z, pv.w + bv.w};
                float g[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) g[j] = a.silu ? pl[j] * sigmoidf_(pl[j]) : pl[j];
                e[i] = make_float4(xv.x * g[0], xv.y * g[1], xv.z * g[2], xv.w * g[3]);
                sum += e[i].x + e[i].y + e[i].z + e[i].w;
            }
        }
        const float mean = warp_sum(sum) * invD;
        float vs = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = (i * 32 + lane) * 4;
            if (i < nv && d < a.D) {
                float dx = e[i].x - mean, dy = e[i].y - mean, dz = e[i].z - mean, dw = e[i].w - mean;
                vs += dx * dx + dy * dy + dz * dz + dw * dw;
            }
        }
        const float var = warp_sum(vs) * invD;
        const float rs = 1.0f / sqrtf(var + a.eps);
        if (lane == 0) {
            a.mu[row] = mean;
            a.rstd[row] = rs;
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = (i * 32 + lane) * 4;
            if (i < nv && d < a.D) {
                float4 w = *reinterpret_cast<const float4*>(a.ln_w + d);
                float4 bb = *reinterpret_cast<const float4*>(a.ln_b + d);
                float4 o;
                o.x = (e[i].x - mean) * rs * w.x + bb.x;
                o.y = (e[i].y - mean) * rs * w.y + bb.y;
                o.z = (e[i].z - mean) * rs * w.z + bb.z;
                o.w = (e[i].w - mean) * rs * w.w + bb.w;
                st4_dyn(a.y, a.y_dt, (size_t)row * a.D + d, o);
            }
        }
    }
}

struct QGateBwdArgs {
    const void* dy; int dy_dt;
    const void* x; int x_dt;
    const void* p; int p_dt;
    const float* bias; const float* ln_w; const float* mu; const float* rstd;
    float* dx; float* dp;
    float* part;  // [gridDim.x][3][D]  (dbias, dln_w, dln_b) partial column sums
    long long rows; int D; int silu;
};

// dynamic smem: float red[QG_WARPS][3][D]
template <int NV>
__global__ void __launch_bounds__(QG_WARPS * 32, NV <= 4 ? 2 : 1) k_qgate_bwd(QGateBwdArgs a) {
    extern __shared__ float red[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    constexpr int nv = NV;
    const float invD = 1.0f / (float)a.D;
    float4 acc_b[NV], acc_w[NV], acc_lb[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) acc_b[i] = acc_w[i] = acc_lb[i] = make_float4(0.f, 0.f, 0.f, 0.f);

    for (long long row = (long long)blockIdx.x * QG_WARPS + warp; row < a.rows; row += (long long)gridDim.x * QG_WARPS) {
        const float mean = a.mu[row];
        const float rs = a.rstd[row];
        float4 dxh[NV], xh[NV], gx[NV], gg[NV];  // dx_hat, x_hat, x*dsilu, gate
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = (i * 32 + lane) * 4;
            dxh[i] = xh[i] = gx[i] = gg[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < nv && d < a.D) {
                float4 dyv = ld4_dyn_f32(a.dy, a.dy_dt, (size_t)row * a.D + d);
                float4 xv = ld4_dyn_f32(a.x, a.x_dt, (size_t)row * a.D + d);
                float4 pv = ld4_dyn_f32(a.p, a.p_dt, (size_t)row * a.D + d);
                float4 bv = *reinterpret_cast<const float4*>(a.bias + d);
                float4 lw = *reinterpret_cast<const float4*>(a.ln_w + d);
                float dyy[4] = {dyv.x, dyv.y, dyv.z, dyv.w};
                float xx[4] = {xv.x, xv.y, xv.z, xv.w};
                float pl[4] = {pv.x + bv.x, pv.y + bv.y, pv.z + bv.z, pv.w + bv.w};
                float lww[4] = {lw.x, lw.y, lw.z, lw.w};
                float o_dxh[4], o_xh[4], o_gx[4], o_g[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float g, dsl;
                    if (a.silu) {
                        float sg = sigmoidf_(pl[j]);
                        g = pl[j] * sg;
                        dsl = g + sg * (1.0f - g);
                    } else {
                        g = pl[j];
                        dsl = 1.0f;
                    }
                    float xe = xx[j] * g;
                    o_xh[j] = (xe - mean) * rs;
                    o_dxh[j] = dyy[j] * lww[j];
                    o_gx[j] = xx[j] * dsl;
                    o_g[j] = g;
                    s1 += o_dxh[j];
                    s2 += o_dxh[j] * o_xh[j];
                }
                dxh[i] = make_float4(o_dxh[0], o_dxh[1], o_dxh[2], o_dxh[3]);
                xh[i] = make_float4(o_xh[0], o_xh[1], o_xh[2], o_xh[3]);
                gx[i] = make_float4(o_gx[0], o_gx[1], o_gx[2], o_gx[3]);
                gg[i] = make_float4(o_g[0], o_g[1], o_g[2], o_g[3]);
                acc_w[i].x += dyy[0] * o_xh[0]; acc_w[i].y += dyy[1] * o_xh[1];
                acc_w[i].z += dyy[2] * o_xh[2]; acc_w[i].w += dyy[3] * o_xh[3];
                acc_lb[i].x += dyy[0]; acc_lb[i].y += dyy[1]; acc_lb[i].z += dyy[2]; acc_lb[i].w += dyy[3];
            }
        }
        const float c1 = warp_sum(s1) * invD;
        const float c2 = warp_sum(s2) * invD;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = (i * 32 + lane) * 4;
            if (i < nv && d < a.D) {
                float4 de;
                de.x = (dxh[i].x - c1 - xh[i].x * c2) * rs;
                de.y = (dxh[i].y - c1 - xh[i].y * c2) * rs;
                de.z = (dxh[i].z - c1 - xh[i].z * c2) * rs;
                de.w = (dxh[i].w - c1 - xh[i].w * c2) * rs;
                float4 dxq = make_float4(de.x * gg[i].x, de.y * gg[i].y, de.z * gg[i].z, de.w * gg[i].w);
                float4 dpp = make_float4(de.x * gx[i].x, de.y * gx[i].y, de.z * gx[i].z, de.w * gx[i].w);
                *reinterpret_cast<float4*>(a.dx + (size_t)row * a.D + d) = dxq;
                *reinterpret_cast<float4*>(a.dp + (size_t)row * a.D + d) = dpp;
                acc_b[i].x += dpp.x; acc_b[i].y += dpp.y; acc_b[i].z += dpp.z; acc_b[i].w += dpp.w;
            }
        }
    }
    // CTA reduction of the three column sums (fixed order -> deterministic)
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = (i * 32 + lane) * 4;
        if (i < nv && d < a.D) {
            *reinterpret_cast<float4*>(&red[(warp * 3 + 0) * a.D + d]) = acc_b[i];
            *reinterpret_cast<float4*>(&red[(warp * 3 + 1) * a.D + d]) = acc_w[i];
            *reinterpret_cast<float4*>(&red[(warp * 3 + 2) * a.D + d]) = acc_lb[i];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 3 * a.D; idx += blockDim.x) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < QG_WARPS; ++w) s += red[w * 3 * a.D + idx];
        a.part[(size_t)blockIdx.x * 3 * a.D + idx] = s;
    }
}

// out[j][d] = sum_c part[c][j][d]: a CTA owns 32 columns, its 8 warps split the partials, fixed order -> deterministic
__global__ void __launch_bounds__(256) k_qgate_colsum(const float* __restrict__ part, int nparts, int D, float* dbias, float* dln_w, float* dln_b) {
    __shared__ float red[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int idx = blockIdx.x * 32 + lane;
    float s = 0.f;
    if (idx < 3 * D)
        for (int c = warp; c < nparts; c += 8) s += part[(size_t)c * 3 * D + idx];
    red[warp][lane] = s;
    __syncthreads();
    if (warp == 0 && idx < 3 * D) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[w][lane];
        const int j = idx / D, d = idx % D;
        (j == 0 ? dbias : (j == 1 ? dln_w : dln_b))[d] = t;
    }
}

static int sm_count() {
    int dev = 0, n = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 148;
}

// One wave of resident CTAs: SM count x the kernel's occupancy (a grid-stride loop covers the rows); a larger grid
// would run a partial second wave.  `per_sm_cap` bounds the workspace of the backward.
static constexpr int QG_MAX_CTAS_PER_SM = 8;
template <typename K>
static int qgate_grid(int64_t rows, K kernel, size_t smem) {
    int occ = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, QG_WARPS * 32, smem) != cudaSuccess || occ < 1) occ = 1;
    if (occ > QG_MAX_CTAS_PER_SM) occ = QG_MAX_CTAS_PER_SM;
    const int64_t ctas = (rows + QG_WARPS - 1) / QG_WARPS, cap = (int64_t)sm_count() * occ;
    return (int)(ctas < cap ? (ctas < 1 ? 1 : ctas) : cap);
}

}  // namespace mbema

using namespace mbema;

static int qgate_check(int64_t rows, int64_t D) {
    if (rows < 0 || D < 4) return MBEMA_ERR_SHAPE;
    if (D % 4 != 0 || D > 1024) return MBEMA_ERR_UNSUPPORTED;
    return MBEMA_OK;
}

static bool dt_ok(int dt) { return dt == MBEMA_F32 || dt == MBEMA_BF16; }

extern "C" int mbema_qgate_fwd(const void* x_q, int x_dtype, const void* p_pre, int p_dtype, const float* bias,
                               const float* ln_w, const float* ln_b, float eps, void* Y, int y_dtype, float* mu,
                               float* rstd, int64_t rows, int64_t D, int flags, void* stream) {
    int rc = qgate_check(rows, D);
    if (rc) return rc;
    if (rows == 0) return MBEMA_OK;
    if (!x_q || !p_pre || !bias || !ln_w || !ln_b || !Y || !mu || !rstd) return MBEMA_ERR_NULL;
    if (!dt_ok(x_dtype) || !dt_ok(p_dtype) || !dt_ok(y_dtype)) return MBEMA_ERR_DTYPE;
    if (((uintptr_t)x_q | (uintptr_t)p_pre | (uintptr_t)bias | (uintptr_t)ln_w | (uintptr_t)ln_b | (uintptr_t)Y) & 15)
        return MBEMA_ERR_ALIGN;
    QGateFwdArgs a{x_q, x_dtype, p_pre, p_dtype, bias, ln_w, ln_b, eps, Y, y_dtype, mu, rstd, rows, (int)D,
                   (flags & MBEMA_FLAG_SILU) ? 1 : 0};
    cudaStream_t st = (cudaStream_t)stream;
    if (D <= 128) k_qgate_fwd<1><<<qgate_grid(rows, k_qgate_fwd<1>, 0), QG_WARPS * 32, 0, st>>>(a);
    else if (D <= 256) k_qgate_fwd<2><<<qgate_grid(rows, k_qgate_fwd<2>, 0), QG_WARPS * 32, 0, st>>>(a);
    else if (D <= 512) k_qgate_fwd<4><<<qgate_grid(rows, k_qgate_fwd<4>, 0), QG_WARPS * 32, 0, st>>>(a);
    else k_qgate_fwd<8><<<qgate_grid(rows, k_qgate_fwd<8>, 0), QG_WARPS * 32, 0, st>>>(a);
    return check_launch();
}

extern "C" size_t mbema_qgate_bwd_workspace_bytes(int64_t rows, int64_t D) {
    const int64_t ctas = (rows + QG_WARPS - 1) / QG_WARPS, cap = (int64_t)sm_count() * QG_MAX_CTAS_PER_SM;
    return (size_t)(ctas < cap ? (ctas < 1 ? 1 : ctas) : cap) * 3 * (size_t)D * sizeof(float) + 256;
}

extern "C" int mbema_qgate_bwd(const void* dY, int dy_dtype, const void* x_q, int x_dtype, const void* p_pre,
                               int p_dtype, const float* bias, const float* ln_w, const float* mu, const float* rstd,
                               float* dx_q, float* dp_pre, float* dbias, float* dln_w, float* dln_b, int64_t rows,
                               int64_t D, int flags, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = qgate_check(rows, D);
    if (rc) return rc;
    if (!dbias || !dln_w || !dln_b) return MBEMA_ERR_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    if (rows == 0) {
        MBEMA_CUDA_TRY(cudaMemsetAsync(dbias, 0, D * sizeof(float), st));
        MBEMA_CUDA_TRY(cudaMemsetAsync(dln_w, 0, D * sizeof(float), st));
        MBEMA_CUDA_TRY(cudaMemsetAsync(dln_b, 0, D * sizeof(float), st));
        return MBEMA_OK;
    }
    if (!dY || !x_q || !p_pre || !bias || !ln_w || !mu || !rstd || !dx_q || !dp_pre || !workspace) return MBEMA_ERR_NULL;
    if (!dt_ok(dy_dtype) || !dt_ok(x_dtype) || !dt_ok(p_dtype)) return MBEMA_ERR_DTYPE;
    if (((uintptr_t)dY | (uintptr_t)x_q | (uintptr_t)p_pre | (uintptr_t)bias | (uintptr_t)ln_w | (uintptr_t)dx_q |
         (uintptr_t)dp_pre) & 15)
        return MBEMA_ERR_ALIGN;
    if (workspace_bytes < mbema_qgate_bwd_workspace_bytes(rows, D)) return MBEMA_ERR_WORKSPACE;
    float* part = (float*)(((uintptr_t)workspace + 255) / 256 * 256);
    int grid = 1;
    QGateBwdArgs a{dY, dy_dtype, x_q, x_dtype, p_pre, p_dtype, bias, ln_w, mu, rstd, dx_q, dp_pre, part, rows, (int)D,
                   (flags & MBEMA_FLAG_SILU) ? 1 : 0};
    const size_t smem = (size_t)QG_WARPS * 3 * D * sizeof(float);
#define MBEMA_QG_BWD(NV_)                                                                                        \
    do {                                                                                                         \
        MBEMA_CUDA_TRY(cudaFuncSetAttribute(k_qgate_bwd<NV_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        grid = qgate_grid(rows, k_qgate_bwd<NV_>, smem);                                                         \
        k_qgate_bwd<NV_><<<grid, QG_WARPS * 32, smem, st>>>(a);                                                  \
    } while (0)
    if (D <= 128) MBEMA_QG_BWD(1);
    else if (D <= 256) MBEMA_QG_BWD(2);
    else if (D <= 512) MBEMA_QG_BWD(4);
    else MBEMA_QG_BWD(8);
#undef MBEMA_QG_BWD
    rc = check_launch();
    if (rc) return rc;
    k_qgate_colsum<<<(unsigned)((3 * D + 31) / 32), 256, 0, st>>>(part, grid, (int)D, dbias, dln_w, dln_b);
    return check_launch();
}
