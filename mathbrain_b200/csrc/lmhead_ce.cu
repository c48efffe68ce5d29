// Row-wise softmax cross-entropy over a chunk of logits, forward and backward in one launch, in place:
//   loss[r] = logsumexp(logits[r, :V]) - logits[r, target[r]],   logits[r, :] <- (softmax(logits[r, :V]) - onehot) * scale
// The chunked tied lm_head (mathbrain/model.py:185-186 computes [B*T, V] logits at once; train.py:320-323 applies the
// masked cross-entropy) runs a library GEMM per chunk of VALID rows, this kernel on the chunk, and two more GEMMs
// (dh = dlogits E, dE += dlogits^T h), so the full logits never exist and masked positions cost nothing.
// HBM-bound: one read and one write of the chunk (the later reads of a row come from L2: a bf16 row is 100 KB).
// Rows have a padded leading dimension (a multiple of 8 elements) so that every row starts 16-byte aligned; the
// padding columns [V, ld) are written as zeros.
#include "common.cuh"

namespace mbema {

constexpr int CE_THREADS = 256;

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// (m, s) <- merge with (m2, s2): maxima in log2 units, sums relative to them
__device__ __forceinline__ void ce_merge(float& m, float& s, float m2, float s2) {
    const float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * ex2_approx(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * ex2_approx(m2 - mn));
    m = mn;
}

template <int DT, int VEC>
__device__ __forceinline__ void ce_load(const void* p, size_t i, float* v) {
    const float4 a = ld4_dyn_f32(p, DT, i);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    if (VEC == 8) {
        const float4 b = ld4_dyn_f32(p, DT, i + 4);
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

// One CTA per row, two sweeps: an online (maximum, sum of exp) per thread over its share of the row, merged across the
// CTA; then the gradient, written over the logits.  The first sweep reads DRAM, the second finds the row (100 KB in
// bf16) in L2; the grid is sized so that the rows in flight fit there.  Full vectors take a path without per-element
// bounds tests, the one-hot term is subtracted afterwards by one thread, exponentials are ex2 of pre-scaled arguments.
template <int DT>
__global__ void __launch_bounds__(CE_THREADS)
k_ce_rows(void* __restrict__ logits, const int64_t* __restrict__ targets, float scale, float* __restrict__ loss_rows,
          int64_t R, int64_t V64, int64_t ld64) {
    constexpr int VEC = (DT == MBEMA_F32) ? 4 : 8;
    constexpr float L2E = 1.4426950408889634f;
    __shared__ float red_m[CE_THREADS / 32], red_s[CE_THREADS / 32];
    __shared__ float bc[2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int V = (int)V64, ld = (int)ld64, Vfull = V / VEC * VEC;
    for (int64_t r = blockIdx.x; r < R; r += gridDim.x) {
        const size_t base = (size_t)r * ld;
        float m = -INFINITY, s = 0.f;          // in units of log2: m = max(x) * log2(e), s = sum 2^(x log2e - m)
        for (int c = tid * VEC; c < V; c += CE_THREADS * VEC) {
            float v[VEC];
            ce_load<DT, VEC>(logits, base + c, v);
            if (c >= Vfull) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) if (c + i >= V) v[i] = -INFINITY;
            }
            float mx = v[0];
#pragma unroll
            for (int i = 1; i < VEC; ++i) mx = fmaxf(mx, v[i]);
            mx = fmaxf(m, mx * L2E);
            float acc = s * ex2_approx(m - mx);        // m = -inf at the start: 0 * 2^(-inf) = 0
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc += ex2_approx(fmaf(v[i], L2E, -mx));
            m = mx; s = acc;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
            ce_merge(m, s, m2, s2);
        }
        if (lane == 0) { red_m[warp] = m; red_s[warp] = s; }
        __syncthreads();
        if (tid == 0) {
            float mm = red_m[0], ss = red_s[0];
            for (int i = 1; i < CE_THREADS / 32; ++i) ce_merge(mm, ss, red_m[i], red_s[i]);
            bc[0] = mm; bc[1] = ss;
            const int64_t t = targets[r];
            const float xt = (t >= 0 && t < V) ? ld_dyn_f32(logits, DT, base + t) : 0.f;
            loss_rows[r] = (t >= 0 && t < V) ? (logf(ss) + mm * (1.0f / L2E) - xt) : 0.f;
        }
        __syncthreads();
        const int64_t t = targets[r];
        const bool has_t = t >= 0 && t < V;
        const float mm = bc[0], inv = has_t ? scale / bc[1] : 0.f;       // a row without a target gets a zero gradient
        for (int c = tid * VEC; c < ld; c += CE_THREADS * VEC) {
            float v[VEC];
            ce_load<DT, VEC>(logits, base + c, v);
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[i] = ex2_approx(fmaf(v[i], L2E, -mm)) * inv;
            if (c >= Vfull) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) if (c + i >= V) v[i] = 0.f;
            }
            if (has_t && (int)t >= c && (int)t < c + VEC) {      // the one-hot term (one thread per row takes this branch)
#pragma unroll
                for (int i = 0; i < VEC; ++i) if (c + i == (int)t) v[i] -= scale;
            }
            st4_dyn(logits, DT, base + c, make_float4(v[0], v[1], v[2], v[3]));
            if (VEC == 8) st4_dyn(logits, DT, base + c + 4, make_float4(v[4], v[5], v[6], v[7]));
        }
        __syncthreads();
    }
}

}  // namespace mbema

using namespace mbema;

extern "C" int mbema_ce_rows(void* logits, int dtype, const int64_t* targets, float scale, float* loss_rows, int64_t R,
                             int64_t V, int64_t ld, void* stream) {
    if (R < 0 || V <= 0 || ld < V || ld % 8 != 0) return MBEMA_ERR_SHAPE;
    if (R == 0) return MBEMA_OK;
    if (!logits || !targets || !loss_rows) return MBEMA_ERR_NULL;
    if (dtype != MBEMA_F32 && dtype != MBEMA_BF16) return MBEMA_ERR_DTYPE;
    if ((uintptr_t)logits & 15) return MBEMA_ERR_ALIGN;
    int dev = 0, sms = 148;
    MBEMA_CUDA_TRY(cudaGetDevice(&dev));
    MBEMA_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t cap = (int64_t)sms * 4;        // rows in flight: 592 x 100 KB stay below the L2 capacity
    const int grid = (int)(R < cap ? R : cap);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == MBEMA_F32) k_ce_rows<MBEMA_F32><<<grid, CE_THREADS, 0, st>>>(logits, targets, scale, loss_rows, R, V, ld);
    else k_ce_rows<MBEMA_BF16><<<grid, CE_THREADS, 0, st>>>(logits, targets, scale, loss_rows, R, V, ld);
    return check_launch();
}
