// Streaming decode on the tensor cores (MBEMA_MODE_TC_BF16, N = 64): attention of ONE query per sequence over the
// slots seen so far.  Rows of the tile are SLOTS here (a thread per slot), so the softmax runs across threads; it is
// split in three launches instead of an online update:
//   pass 1   per (sequence, 128-slot tile, head pair): decayed state tile -> tcgen05.mma -> gate -> score s[b,h,k]
//   softmax  per (sequence, head): probabilities over all V_total slots (the never-seen ones add exp(0 - max) each)
//   pass 2   same tile product again, P.V: the bf16 tile (p * gate * E_v)[k, d] is summed over its 128 slots by a
//            second tcgen05.mma against a ones operand (the column-sum trick of the training backward) and added to
//            O[b,h,:] with fp32 atomics.
// One tile per CTA, no pipeline inside the CTA: eight warps, several CTAs per SM overlap each other's latencies.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace mbema {
namespace dtc {

using namespace ptx;

static constexpr int TM = 128, HD = 64, HPC = 2, N = 64, ACC_COLS = HPC * HD, THREADS = 256;
static constexpr int ATOM_BYTES = TM * 128;

struct Args {
    const void* q; int q_dt;
    const void* Ek; const void* Ev; int e_dt;
    const float* W; const float* rhos;
    const float* state; const int* last_t; const int* active; const int* n_active;
    float* scores;                 // [B, H, Kcap]: scores after pass 1, probabilities after the softmax
    float* O;                      // [B, H, 64]
    int B, H, V, Kcap, t_now;
    float v_total;
    int listed_only;
};

__device__ __forceinline__ int sw128_off(int row, int col) {
    return row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1));
}

struct Bars { uint64_t acc_full; uint64_t pv_done; uint32_t tmem_base; int abort_flag; };

// dynamic smem (base aligned to 1024): A 16 KB | B 16 KB | Vg 32 KB | ones 2 KB | q 512 B | l2r 256 B | bars
template <int PASS, bool SILU>
__global__ void __launch_bounds__(THREADS) k_decode_tc(Args a, int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* A_sh = sm;
    unsigned char* B_sh = sm + ATOM_BYTES;
    unsigned char* V_sh = sm + 2 * ATOM_BYTES;                 // [head][128 k][64 d] bf16, MN-major operand of pass 2
    unsigned char* ones_sh = sm + 4 * ATOM_BYTES;
    float* q_sh = reinterpret_cast<float*>(sm + 4 * ATOM_BYTES + 2048);            // q / sqrt(hd) of the two heads
    float* l2r_sh = reinterpret_cast<float*>(sm + 4 * ATOM_BYTES + 2048 + 512);
    Bars* bars = reinterpret_cast<Bars*>(sm + 4 * ATOM_BYTES + 2048 + 768);
    volatile int* abort_flag = &bars->abort_flag;

    const int tile = blockIdx.x, hp = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wg = tid >> 7, row = tid & 127;
    const int D = a.H * HD;
    const int na = min(a.n_active[b], a.Kcap);
    if (tile * TM >= na) return;                                // uniform per CTA
    const int h = hp * HPC + wg;
    const int k = tile * TM + row;
    const bool ok = k < na;
    const int v = ok ? a.active[(size_t)b * a.Kcap + k] : 0;

    if (tid == 0) {
        mbar_init(&bars->acc_full, 1);
        mbar_init(&bars->pv_done, 1);
        bars->abort_flag = *reinterpret_cast<volatile int*>(status);
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc(&bars->tmem_base, 128);
        tmem_relinquish();
    }
    // slot-embedding row of this thread's slot for its head: 64 bf16 / fp32 values, fetched before anything waits
    float er[HD];
    {
        const void* src = (PASS == 1) ? a.Ek : a.Ev;
        const size_t off = (size_t)v * D + h * HD;
#pragma unroll
        for (int i = 0; i < HD; i += 4) {
            const float4 x = ld4_dyn_f32(src, a.e_dt, off + i);
            er[i] = x.x; er[i + 1] = x.y; er[i + 2] = x.z; er[i + 3] = x.w;
        }
    }
    const float prob = (PASS == 2 && ok) ? a.scores[((size_t)b * a.H + h) * a.Kcap + k] : 0.f;
    {
        const float wscale = SILU ? 0.5f : 1.0f;
        for (int i = tid; i < N * ACC_COLS; i += THREADS) {
            const int n = i / ACC_COLS, dd = i % ACC_COLS;
            *reinterpret_cast<__nv_bfloat16*>(B_sh + sw128_off(dd, n)) = __float2bfloat16(a.W[(size_t)n * D + hp * ACC_COLS + dd] * wscale);
        }
        if (PASS == 2)
            for (int i = tid; i < 1024; i += THREADS) reinterpret_cast<__nv_bfloat16*>(ones_sh)[i] = __float2bfloat16(1.0f);
        if (tid < N) l2r_sh[tid] = log2f(a.rhos[tid]);
        if (tid < ACC_COLS) q_sh[tid] = ld_dyn_f32(a.q, a.q_dt, ((size_t)b * a.H + hp * HPC) * HD + tid) * 0.125f;
    }
    __syncthreads();
    // decayed state tile: row = slot, this thread fills channels [32 wg, 32 wg + 32)
    {
        const float dt = ok ? (float)(a.t_now - a.last_t[(size_t)b * a.V + v]) : 0.f;
        const float* srow = a.state + ((size_t)b * a.V + v) * N + 32 * wg;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            uint4 pk = make_uint4(0u, 0u, 0u, 0u);
            if (ok) {
                const float4 s0 = __ldg(reinterpret_cast<const float4*>(srow + cc * 8));
                const float4 s1 = __ldg(reinterpret_cast<const float4*>(srow + cc * 8 + 4));
                const float* lr = l2r_sh + 32 * wg + cc * 8;
                pk.x = pack_bf16x2(s0.x * exp2f(dt * lr[0]), s0.y * exp2f(dt * lr[1]));
                pk.y = pack_bf16x2(s0.z * exp2f(dt * lr[2]), s0.w * exp2f(dt * lr[3]));
                pk.z = pack_bf16x2(s1.x * exp2f(dt * lr[4]), s1.y * exp2f(dt * lr[5]));
                pk.w = pack_bf16x2(s1.z * exp2f(dt * lr[6]), s1.w * exp2f(dt * lr[7]));
            }
            *reinterpret_cast<uint4*>(A_sh + row * 128 + (((4 * wg + cc) ^ (row & 7)) << 4)) = pk;
        }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;
    if (tid == 0 && !bars->abort_flag) {
        const uint32_t idesc = umma_idesc_bf16(TM, ACC_COLS, 0, 0);
        const uint64_t da = umma_desc_k_sw128(smem_u32(A_sh)), db = umma_desc_k_sw128(smem_u32(B_sh));
#pragma unroll
        for (int k16 = 0; k16 < 4; ++k16)
            umma_bf16_ss(tmem_base, da + (uint64_t)((k16 * 32) >> 4), db + (uint64_t)((k16 * 32) >> 4), idesc, k16 != 0 ? 1u : 0u);
        umma_commit(&bars->acc_full);
    }
    if (!bars->abort_flag) mbar_wait(&bars->acc_full, 0u, abort_flag);
    tc_fence_after_sync();
    const uint32_t t_acc = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(wg * HD);
    const float* qh = q_sh + wg * HD;
    if (PASS == 1) {
        float sp[2] = {0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float pre[32];
            tmem_ld_32x32b_x32(t_acc + c * 32, pre);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                const float h0 = pre[j], h1 = pre[j + 1];
                const float g0 = SILU ? fmaf(h0, tanh_approx(h0), h0) : h0;
                const float g1 = SILU ? fmaf(h1, tanh_approx(h1), h1) : h1;
                sp[0] = fmaf(g0 * qh[c * 32 + j], er[c * 32 + j], sp[0]);
                sp[1] = fmaf(g1 * qh[c * 32 + j + 1], er[c * 32 + j + 1], sp[1]);
            }
        }
        if (ok) a.scores[((size_t)b * a.H + h) * a.Kcap + k] = sp[0] + sp[1];
    } else {
        unsigned char* vrow = V_sh + wg * ATOM_BYTES + row * 128;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float pre[32];
            tmem_ld_32x32b_x32(t_acc + c * 32, pre);
            tmem_wait_ld();
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
                uint32_t w[4];
#pragma unroll
                for (int pr = 0; pr < 4; ++pr) {
                    const int j = j8 * 8 + pr * 2;
                    const float h0 = pre[j], h1 = pre[j + 1];
                    const float g0 = SILU ? fmaf(h0, tanh_approx(h0), h0) : h0;
                    const float g1 = SILU ? fmaf(h1, tanh_approx(h1), h1) : h1;
                    w[pr] = pack_bf16x2(prob * g0 * er[c * 32 + j], prob * g1 * er[c * 32 + j + 1]);
                }
                st_shared_v4(vrow + (((c * 4 + j8) ^ (row & 7)) << 4), w[0], w[1], w[2], w[3]);
            }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();                    // every warp has read its accumulators and written its part of the tile
        tc_fence_after_sync();
        if (tid == 0 && !bars->abort_flag) {
            const uint32_t idesc = umma_idesc_bf16(ACC_COLS, 16, 1, 0);
            const uint64_t dv = umma_desc_mn_sw128(smem_u32(V_sh), ATOM_BYTES, 1024), d1 = umma_desc_k_sw128(smem_u32(ones_sh));
#pragma unroll
            for (int ks = 0; ks < TM / 16; ++ks)
                umma_bf16_ss(tmem_base, dv + (uint64_t)(ks * (2048 >> 4)), d1, idesc, ks != 0 ? 1u : 0u);   // reuses the gate columns
            umma_commit(&bars->pv_done);
        }
        if (!bars->abort_flag) mbar_wait(&bars->pv_done, 0u, abort_flag);
        tc_fence_after_sync();
        if (wg == 0) {                      // lane = output column d of the head pair
            float x;
            {
                uint32_t r;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(tmem_base + ((uint32_t)((warp & 3) * 32) << 16)) : "memory");
                tmem_wait_ld();
                x = __uint_as_float(r);
            }
            atomicAdd(a.O + ((size_t)b * a.H + hp * HPC) * HD + row, x);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 128);
    }
    if (tid == 0 && bars->abort_flag) atomicExch(status, 1);
}

// probabilities over all V_total slots, in place: scores[b,h,k] <- exp(s - m) / l
__global__ void __launch_bounds__(256) k_decode_softmax(Args a) {
    __shared__ float red[8];
    __shared__ float bc;
    const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    const int na = min(a.n_active[b], a.Kcap);
    float* s = a.scores + ((size_t)b * a.H + h) * a.Kcap;
    const float rest = a.listed_only ? 0.f : fmaxf(a.v_total - (float)na, 0.f);
    float m = rest > 0.f ? 0.f : -INFINITY;
    for (int k = tid; k < na; k += 256) m = fmaxf(m, s[k]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();
    if (tid == 0) { float x = red[0]; for (int i = 1; i < 8; ++i) x = fmaxf(x, red[i]); bc = x; }
    __syncthreads();
    m = bc;
    float l = 0.f;
    for (int k = tid; k < na; k += 256) l += __expf(s[k] - m);
    l = warp_sum(l);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = l;
    __syncthreads();
    if (tid == 0) { float x = rest > 0.f ? rest * __expf(-m) : 0.f; for (int i = 0; i < 8; ++i) x += red[i]; bc = x; }
    __syncthreads();
    const float inv = bc > 0.f ? 1.0f / bc : 0.f;
    for (int k = tid; k < na; k += 256) s[k] = __expf(s[k] - m) * inv;
}

}  // namespace dtc
}  // namespace mbema

using namespace mbema;

extern "C" size_t mbema_decode_attend_tc_workspace_bytes(int64_t B, int64_t H, int64_t Kcap) {
    return 512 + (size_t)B * H * Kcap * sizeof(float);
}

extern "C" int mbema_decode_attend_tc(const void* q, int q_dtype, const void* E_k, const void* E_v, int e_dtype,
                                      const float* W_pe, const float* rhos, const float* state, const int32_t* last_t,
                                      const int32_t* active, const int32_t* n_active, float* O, int64_t B, int64_t H,
                                      int64_t hd, int64_t V, int64_t N, int64_t Kcap, int64_t t_now, int64_t V_total,
                                      int flags, void* workspace, size_t workspace_bytes, void* stream) {
    if (B < 0 || H < 1 || V < 1 || N < 1 || Kcap < 1) return MBEMA_ERR_SHAPE;
    if (hd != 64 || N != 64 || (H % 2) != 0 || B > 65535 || H > 65535) return MBEMA_ERR_UNSUPPORTED;
    if (B == 0) return MBEMA_OK;
    if (!q || !E_k || !E_v || !W_pe || !rhos || !state || !last_t || !active || !n_active || !O || !workspace) return MBEMA_ERR_NULL;
    if ((q_dtype != MBEMA_F32 && q_dtype != MBEMA_BF16) || (e_dtype != MBEMA_F32 && e_dtype != MBEMA_BF16)) return MBEMA_ERR_DTYPE;
    if (((uintptr_t)E_k | (uintptr_t)E_v) & 15) return MBEMA_ERR_ALIGN;
    if (workspace_bytes < mbema_decode_attend_tc_workspace_bytes(B, H, Kcap)) return MBEMA_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    int* status = reinterpret_cast<int*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
    dtc::Args a{q, q_dtype, E_k, E_v, e_dtype, W_pe, rhos, state, last_t, active, n_active,
                reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(status) + 256), O,
                (int)B, (int)H, (int)V, (int)Kcap, (int)t_now, (float)V_total, (flags & MBEMA_FLAG_LISTED_ONLY) ? 1 : 0};
    MBEMA_CUDA_TRY(cudaMemsetAsync(status, 0, 256, st));
    MBEMA_CUDA_TRY(cudaMemsetAsync(O, 0, (size_t)B * H * hd * sizeof(float), st));
    const int smem = 4 * dtc::ATOM_BYTES + 2048 + 768 + 64 + 1024;
    dim3 grid((unsigned)((Kcap + dtc::TM - 1) / dtc::TM), (unsigned)(H / 2), (unsigned)B);
    const bool silu = (flags & MBEMA_FLAG_SILU) != 0;
#define MBEMA_DECODE_LAUNCH(P_, S_)                                                                                    \
    do {                                                                                                              \
        MBEMA_CUDA_TRY(cudaFuncSetAttribute(dtc::k_decode_tc<P_, S_>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
        dtc::k_decode_tc<P_, S_><<<grid, dtc::THREADS, smem, st>>>(a, status);                                        \
    } while (0)
    if (silu) MBEMA_DECODE_LAUNCH(1, true); else MBEMA_DECODE_LAUNCH(1, false);
    int rc = check_launch();
    if (rc) return rc;
    dtc::k_decode_softmax<<<dim3((unsigned)H, (unsigned)B), 256, 0, st>>>(a);
    rc = check_launch();
    if (rc) return rc;
    if (silu) MBEMA_DECODE_LAUNCH(2, true); else MBEMA_DECODE_LAUNCH(2, false);
#undef MBEMA_DECODE_LAUNCH
    return check_launch();
}
