// Streaming decode with resident per-sequence slot state (O(1) state per token).
//
// The reference has no decode loop; one decode step is one iteration of the loop body of its PyTorch attention
// (mathbrain/flash_ema_attention.py:46-82) plus the per-token state update of the query scan
// (mathbrain/triton_ema_query.py:36-64), with the [V, N] state kept in HBM between steps and decayed lazily:
//     state[v]  = value of slot v right after its last update,   last_t[v] = step of that update (-1: never)
//     M_t[v]    = state[v] * rho^(t - last_t[v])                 (what step t sees; 0 for never-seen slots)
// `attend` reads the slots seen so far (a per-sequence list) and must run BEFORE `update` of the same step.
// fp32 arithmetic on the CUDA cores; one CTA per (sequence, head), threads = 64 slots x 4 column groups.
#include "common.cuh"

namespace mbema {

static constexpr int DC_SLOTS = 64;
static constexpr int DC_THREADS = DC_SLOTS * 4;
static constexpr int DC_HD = 64;

struct DecodeArgs {
    const void* q; int q_dt;              // [B, H, 64]
    const void* Ek; const void* Ev; int e_dt;   // [V, H*64] shared by all sequences
    const float* W; const float* rhos;    // [N, H*64], [N]
    const float* state; const int* last_t;      // [B, V, N], [B, V]
    const int* active; const int* n_active;     // [B, Kcap], [B]
    float* O;                             // [B, H, 64]
    int B, H, V, N, Kcap, t_now;
    const int* t_dev;              // when not null: the step number is read from device memory (graph replays)
    float v_total;
    int silu, listed_only;
};

// dynamic smem: W_sh[N][64] | A_sh[64][N+1] | l2r_sh[N] | red[(64)*(2+16)*4]
__global__ void __launch_bounds__(DC_THREADS) k_decode_attend(DecodeArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int N = a.N, ldA = N + 1;
    float* W_sh = smem;
    float* A_sh = W_sh + N * DC_HD;
    float* l2r_sh = A_sh + ((DC_SLOTS * ldA + 3) & ~3);
    float* red = l2r_sh + ((N + 3) & ~3);        // [DC_THREADS][18]
    const int h = blockIdx.x, b = blockIdx.y;
    const int tid = threadIdx.x;
    const int sr = tid >> 2, dg = tid & 3;
    const int D = a.H * DC_HD;
    for (int i = tid; i < N * DC_HD; i += DC_THREADS) W_sh[i] = a.W[(size_t)(i / DC_HD) * D + h * DC_HD + (i % DC_HD)];
    for (int i = tid; i < N; i += DC_THREADS) l2r_sh[i] = log2f(a.rhos[i]);
    float q[16], o[16];
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
        float4 v = ld4_dyn_f32(a.q, a.q_dt, ((size_t)b * a.H + h) * DC_HD + dg * 16 + i);
        q[i] = v.x * 0.125f; q[i + 1] = v.y * 0.125f; q[i + 2] = v.z * 0.125f; q[i + 3] = v.w * 0.125f;
        o[i] = o[i + 1] = o[i + 2] = o[i + 3] = 0.f;
    }
    const int na = min(a.n_active[b], a.Kcap);
    float m = -INFINITY, l = 0.f;
    __syncthreads();
    for (int k0 = 0; k0 < na; k0 += DC_SLOTS) {
        const int k = k0 + sr;
        const bool ok = k < na;
        const int v = ok ? a.active[(size_t)b * a.Kcap + k] : 0;
        {   // decayed state row of this thread's slot (columns dg, dg+4, ...)
            const float dt = ok ? (float)((a.t_dev ? *a.t_dev : a.t_now) - a.last_t[(size_t)b * a.V + v]) : 0.f;
            const float* srow = a.state + ((size_t)b * a.V + v) * N;
            for (int n = dg; n < N; n += 4) A_sh[sr * ldA + n] = ok ? srow[n] * exp2f(dt * l2r_sh[n]) : 0.f;
        }
        float ek[16], ev[16];
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
            const size_t eoff = (size_t)v * D + h * DC_HD + dg * 16 + i;
            float4 v1 = ld4_dyn_f32(a.Ek, a.e_dt, eoff), v2 = ld4_dyn_f32(a.Ev, a.e_dt, eoff);
            ek[i] = v1.x; ek[i + 1] = v1.y; ek[i + 2] = v1.z; ek[i + 3] = v1.w;
            ev[i] = v2.x; ev[i + 1] = v2.y; ev[i + 2] = v2.z; ev[i + 3] = v2.w;
        }
        __syncthreads();
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
        const float* arow = A_sh + sr * ldA;
        const float* wcol = W_sh + dg * 16;
#pragma unroll 4
        for (int n = 0; n < N; ++n) {
            const float av = arow[n];
            const float4* wp = reinterpret_cast<const float4*>(wcol + n * DC_HD);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float4 wv = wp[j];
                acc[4 * j] = fmaf(av, wv.x, acc[4 * j]);
                acc[4 * j + 1] = fmaf(av, wv.y, acc[4 * j + 1]);
                acc[4 * j + 2] = fmaf(av, wv.z, acc[4 * j + 2]);
                acc[4 * j + 3] = fmaf(av, wv.w, acc[4 * j + 3]);
            }
        }
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float g = a.silu ? acc[i] * sigmoidf_(acc[i]) : acc[i];
            acc[i] = g;
            part = fmaf(g * q[i], ek[i], part);
        }
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        if (ok) {
            const float m_new = fmaxf(m, part);
            const float alpha = __expf(m - m_new);
            const float p = __expf(part - m_new);
            l = l * alpha + p;
            m = m_new;
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = fmaf(p, acc[i] * ev[i], o[i] * alpha);
        }
        __syncthreads();
    }
    // merge the 64 per-thread softmax states that share a column group
    float* mine = red + tid * 18;
    mine[0] = m; mine[1] = l;
#pragma unroll
    for (int i = 0; i < 16; ++i) mine[2 + i] = o[i];
    __syncthreads();
    if (sr == 0) {
        float M = -INFINITY;
        for (int s = 0; s < DC_SLOTS; ++s) M = fmaxf(M, red[(s * 4 + dg) * 18]);
        const float rest = a.listed_only ? 0.f : fmaxf(a.v_total - (float)na, 0.f);
        if (rest > 0.f) M = fmaxf(M, 0.f);
        float L = (rest > 0.f) ? rest * __expf(-M) : 0.f;
        float out[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) out[i] = 0.f;
        for (int s = 0; s < DC_SLOTS; ++s) {
            const float* r = red + (s * 4 + dg) * 18;
            if (r[1] > 0.f) {
                const float w = __expf(r[0] - M);
                L += r[1] * w;
#pragma unroll
                for (int i = 0; i < 16; ++i) out[i] = fmaf(r[2 + i], w, out[i]);
            }
        }
        const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) a.O[((size_t)b * a.H + h) * DC_HD + dg * 16 + i] = out[i] * inv;
    }
}

// one warp per sequence: query-side state of the new token, then the slot update
__global__ void k_decode_update(const long long* __restrict__ tok, const float* __restrict__ rhos, float* __restrict__ state,
                                int* __restrict__ last_t, int* __restrict__ active, int* __restrict__ n_active,
                                float* __restrict__ C_q, int* __restrict__ overflow, int B, int V, int N, int Kcap, int t_host,
                                const int* __restrict__ t_dev) {
    const int t_now = t_dev ? *t_dev : t_host;
    const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (b >= B) return;
    const long long v = tok[b];
    if (v < 0 || v >= V) { if (lane == 0) atomicExch(overflow, 2); return; }
    const int lt = last_t[(size_t)b * V + v];
    const double dt = (double)(t_now - lt);
    for (int n = lane; n < N; n += 32) {
        float c = 0.f;
        if (lt >= 0) c = state[((size_t)b * V + v) * N + n] * (float)exp2(dt * log2((double)rhos[n]));
        C_q[(size_t)b * N + n] = c;
        state[((size_t)b * V + v) * N + n] = c + 1.0f;
    }
    __syncwarp();
    if (lane == 0) {
        if (lt < 0) {
            const int pos = n_active[b];
            if (pos < Kcap) { active[(size_t)b * Kcap + pos] = (int)v; n_active[b] = pos + 1; }
            else atomicExch(overflow, 1);
        }
        last_t[(size_t)b * V + v] = t_now;
    }
}

__global__ void k_decode_advance(int* t_dev) { *t_dev += 1; }

}  // namespace mbema

using namespace mbema;

extern "C" int mbema_decode_attend(const void* q, int q_dtype, const void* E_k, const void* E_v, int e_dtype,
                                   const float* W_pe, const float* rhos, const float* state, const int32_t* last_t,
                                   const int32_t* active, const int32_t* n_active, float* O, int64_t B, int64_t H,
                                   int64_t hd, int64_t V, int64_t N, int64_t Kcap, int64_t t_now, int64_t V_total,
                                   int flags, const int32_t* t_now_dev, void* stream) {
    if (B < 0 || H < 1 || V < 1 || N < 1 || Kcap < 1) return MBEMA_ERR_SHAPE;
    if (hd != 64 || N > 128 || B > 65535 || H > 65535) return MBEMA_ERR_UNSUPPORTED;
    if (B == 0) return MBEMA_OK;
    if (!q || !E_k || !E_v || !W_pe || !rhos || !state || !last_t || !active || !n_active || !O) return MBEMA_ERR_NULL;
    if ((q_dtype != MBEMA_F32 && q_dtype != MBEMA_BF16) || (e_dtype != MBEMA_F32 && e_dtype != MBEMA_BF16)) return MBEMA_ERR_DTYPE;
    if (((uintptr_t)q | (uintptr_t)E_k | (uintptr_t)E_v) & 15) return MBEMA_ERR_ALIGN;
    DecodeArgs a{q, q_dtype, E_k, E_v, e_dtype, W_pe, rhos, state, last_t, active, n_active, O,
                 (int)B, (int)H, (int)V, (int)N, (int)Kcap, (int)t_now, t_now_dev, (float)V_total,
                 (flags & MBEMA_FLAG_SILU) ? 1 : 0, (flags & MBEMA_FLAG_LISTED_ONLY) ? 1 : 0};
    const size_t smem = ((size_t)N * DC_HD + ((DC_SLOTS * (N + 1) + 3) & ~3) + ((N + 3) & ~3) + DC_THREADS * 18) * 4;
    MBEMA_CUDA_TRY(cudaFuncSetAttribute(k_decode_attend, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)H, (unsigned)B);
    k_decode_attend<<<grid, DC_THREADS, smem, (cudaStream_t)stream>>>(a);
    return check_launch();
}

extern "C" int mbema_decode_update(const int64_t* tok, const float* rhos, float* state, int32_t* last_t, int32_t* active,
                                   int32_t* n_active, float* C_q, int32_t* overflow, int64_t B, int64_t V, int64_t N,
                                   int64_t Kcap, int64_t t_now, const int32_t* t_now_dev, void* stream) {
    if (B < 0 || V < 1 || N < 1 || Kcap < 1) return MBEMA_ERR_SHAPE;
    if (N > 128) return MBEMA_ERR_UNSUPPORTED;
    if (B == 0) return MBEMA_OK;
    if (!tok || !rhos || !state || !last_t || !active || !n_active || !C_q || !overflow) return MBEMA_ERR_NULL;
    k_decode_update<<<(unsigned)((B + 3) / 4), 128, 0, (cudaStream_t)stream>>>((const long long*)tok, rhos, state, last_t, active,
                                                                           n_active, C_q, overflow, (int)B, (int)V, (int)N,
                                                                           (int)Kcap, (int)t_now, t_now_dev);
    return check_launch();
}

extern "C" int mbema_decode_advance(int32_t* t_now_dev, void* stream) {
    if (!t_now_dev) return MBEMA_ERR_NULL;
    k_decode_advance<<<1, 1, 0, (cudaStream_t)stream>>>(t_now_dev);
    return check_launch();
}
