// Row-wise softmax cross-entropy over a chunk of logits, forward and backward in one launch, in place:
//   loss[r] = logsumexp(logits[r, :V]) - logits[r, target[r]],   logits[r, :] <- (softmax(logits[r, :V]) - onehot) * scale
// The chunked tied lm_head (mathbrain/model.py:185-186 computes [B*T, V] logits at once; train.py:320-323 applies the
// masked cross-entropy) runs a library GEMM per chunk of VALID rows, this kernel on the chunk, and two more GEMMs
// (dh = dlogits E, dE += dlogits^T h), so the full logits never exist and masked positions cost nothing.
// HBM-bound: one read and one write of the chunk (the second read of a row comes from L2: a bf16 row is 100 KB).
// Rows have a padded leading dimension (a multiple of 8 elements) so that every row starts 16-byte aligned; the
// padding columns [V, ld) are written as zeros.
#include "common.cuh"

namespace mbema {

constexpr int CE_THREADS = 256;

__device__ __forceinline__ void ce_merge(float& m, float& s, float m2, float s2) {
    const float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mn));
    m = mn;
}

template <int DT>
__global__ void __launch_bounds__(CE_THREADS)
k_ce_rows(void* __restrict__ logits, const int64_t* __restrict__ targets, float scale, float* __restrict__ loss_rows,
          int64_t R, int64_t V, int64_t ld) {
    constexpr int VEC = (DT == MBEMA_F32) ? 4 : 8;
    __shared__ float red_m[CE_THREADS / 32], red_s[CE_THREADS / 32];
    __shared__ float bc[2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int64_t r = blockIdx.x; r < R; r += gridDim.x) {
        const size_t base = (size_t)r * ld;
        float m = -INFINITY, s = 0.f;
        for (int64_t c = (int64_t)tid * VEC; c < V; c += (int64_t)CE_THREADS * VEC) {
            float v[VEC];
            const float4 a = ld4_dyn_f32(logits, DT, base + c);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            if (VEC == 8) {
                const float4 b = ld4_dyn_f32(logits, DT, base + c + 4);
                v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            }
            float mx = m;
#pragma unroll
            for (int i = 0; i < VEC; ++i) if (c + i < V) mx = fmaxf(mx, v[i]);
            float acc = (m == -INFINITY) ? 0.f : s * __expf(m - mx);
#pragma unroll
            for (int i = 0; i < VEC; ++i) if (c + i < V) acc += __expf(v[i] - mx);
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
            loss_rows[r] = (t >= 0 && t < V) ? (logf(ss) + mm - xt) : 0.f;
        }
        __syncthreads();
        const float mm = bc[0], inv = scale / bc[1];
        const int64_t t = targets[r];
        const float on = (t >= 0 && t < V) ? scale : 0.f;       // a row without a target gets a zero gradient
        for (int64_t c = (int64_t)tid * VEC; c < ld; c += (int64_t)CE_THREADS * VEC) {
            float v[VEC];
            const float4 a = ld4_dyn_f32(logits, DT, base + c);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            if (VEC == 8) {
                const float4 b = ld4_dyn_f32(logits, DT, base + c + 4);
                v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            }
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                float gq = (c + i < V && on != 0.f) ? __expf(v[i] - mm) * inv : 0.f;
                if (c + i == t) gq -= on;
                v[i] = gq;
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
    const int64_t cap = (int64_t)sms * 8;
    const int grid = (int)(R < cap ? R : cap);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == MBEMA_F32) k_ce_rows<MBEMA_F32><<<grid, CE_THREADS, 0, st>>>(logits, targets, scale, loss_rows, R, V, ld);
    else k_ce_rows<MBEMA_BF16><<<grid, CE_THREADS, 0, st>>>(logits, targets, scale, loss_rows, R, V, ld);
    return check_launch();
}
