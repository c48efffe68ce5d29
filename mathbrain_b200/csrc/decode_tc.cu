// Streaming decode on the tensor cores (MBEMA_MODE_TC_BF16, N = 64, bf16 slot embeddings): attention of ONE query
// per sequence over the slots seen so far.  Rows of the tile are SLOTS here (a thread per slot), so the softmax runs
// across threads; it is split in three launches instead of an online update:
//   pass 1   per (sequence, head pair, split): decayed state tile -> tcgen05.mma -> gate -> score s[b,h,k]
//   softmax  per (sequence, head): probabilities over all V_total slots (the never-seen ones add exp(0 - max) each)
//   pass 2   same tile product again, then P.V: the bf16 tile (p * gate * E_v)[k, d] is summed over its 128 slots by
//            a second tcgen05.mma against a ones operand (the column-sum trick of the training backward), accumulated
//            in TMEM over all tiles of the CTA and added to O[b,h,:] with one fp32 atomic per column.
// A CTA walks up to MAXT 128-slot tiles.  All gathers (state rows, embedding rows) are cp.async copies two tiles
// ahead into shared-memory rings, so no thread holds a gathered row in registers while it is in flight; the state
// tile of tile i+1 is converted and its UMMA issued before the epilogue of tile i.
#include "common.cuh"
#include <cuda_fp16.h>
#include "sm100_ptx.cuh"

#include <algorithm>
namespace mbema {
namespace dtc {

using namespace ptx;

static constexpr int TM = 128, HD = 64, HPC = 2, N = 64, ACC_COLS = HPC * HD, THREADS = 512, MAXT = 16;
static constexpr int ATOM_BYTES = TM * 128;
static constexpr int STAGE_BYTES = 2 * ATOM_BYTES;            // one state stage (128 rows x 256 B) or one E stage (2 heads)
static constexpr int OFF_B = 0, OFF_A = ATOM_BYTES, OFF_S = 2 * ATOM_BYTES, OFF_E = OFF_S + 2 * STAGE_BYTES,
                     OFF_V = OFF_E + 2 * STAGE_BYTES, OFF_ONES = OFF_V + 2 * ATOM_BYTES, OFF_Q = OFF_ONES + 2048,
                     OFF_L2R = OFF_Q + 512, OFF_IDS = OFF_L2R + 256, OFF_DTS = OFF_IDS + MAXT * TM * 4,
                     OFF_BARS = OFF_DTS + MAXT * TM * 4, SMEM_BYTES = OFF_BARS + 64 + 1024;

struct Args {
    const void* q; int q_dt;
    const __nv_bfloat16* Ek; const __nv_bfloat16* Ev;
    const float* W; const float* rhos;
    const float* state; const int* last_t; const int* active; const int* n_active;
    float* scores;                 // [B, H, Kcap]: scores after pass 1, probabilities after the softmax
    float* O;                      // [B, H, 64]
    int B, H, V, Kcap, t_now, S;   // S: CTAs per (sequence, head pair); CTA s takes tiles s, s + S, ...
    const int* t_dev;              // when not null: the step number is read from device memory (graph replays)
    float v_total;
    int listed_only;
};

__device__ __forceinline__ int sw128_off(int row, int col) {
    return row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <int K>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(K) : "memory"); }

struct Bars { uint64_t acc_full[2]; uint64_t pv_done; uint32_t tmem_base; int abort_flag; };

template <int PASS, bool SILU>
__global__ void __launch_bounds__(THREADS, 1) k_decode_tc(Args a, int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* A_sh = sm + OFF_A;
    unsigned char* B_sh = sm + OFF_B;
    unsigned char* S_st = sm + OFF_S;       // [2][128 rows][16 chunks of 4 floats, chunk ^ (row & 15)]
    unsigned char* E_st = sm + OFF_E;       // [2][head][128 rows][8 chunks of 8 bf16, chunk ^ (row & 7)]
    unsigned char* V_sh = sm + OFF_V;       // [head][128 k][64 d] bf16, MN-major operand of the column sum
    unsigned char* ones_sh = sm + OFF_ONES;
    float* q_sh = reinterpret_cast<float*>(sm + OFF_Q);                 // q / sqrt(hd) of the two heads
    float* l2r_sh = reinterpret_cast<float*>(sm + OFF_L2R);
    int* ids_sh = reinterpret_cast<int*>(sm + OFF_IDS);                 // slot of every row of this CTA's tiles, -1 = none
    float* dts_sh = reinterpret_cast<float*>(sm + OFF_DTS);             // steps since that slot's last update
    Bars* bars = reinterpret_cast<Bars*>(sm + OFF_BARS);
    volatile int* abort_flag = &bars->abort_flag;

    const int split = blockIdx.x, hp = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int cg = tid >> 7, row = tid & 127;                   // column group: head cg >> 1 of the pair, 32-column half cg & 1
    const int hh = cg >> 1, half = cg & 1;
    const int D = a.H * HD;
    const int na = min(a.n_active[b], a.Kcap);
    const int ntile_b = (na + TM - 1) / TM;
    if (split >= ntile_b) return;                               // uniform per CTA
    const int nt = min((ntile_b - split + a.S - 1) / a.S, MAXT);
    const int h = hp * HPC + hh;

    if (tid == 0) {
        mbar_init(&bars->acc_full[0], 1);
        mbar_init(&bars->acc_full[1], 1);
        mbar_init(&bars->pv_done, 1);
        bars->abort_flag = *reinterpret_cast<volatile int*>(status);
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc(&bars->tmem_base, 512);
        tmem_relinquish();
    }
    // B operand values first (independent loads), then the slot ids and their ages (two dependent rounds of loads)
    float4 wv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int g = tid + THREADS * j, n = g >> 5, dd4 = (g & 31) * 4;
        wv[j] = __ldg(reinterpret_cast<const float4*>(a.W + (size_t)n * D + hp * ACC_COLS + dd4));
    }
    const int t_now = a.t_dev ? *a.t_dev : a.t_now;
    int vv[MAXT * TM / THREADS];
#pragma unroll
    for (int j = 0; j < MAXT * TM / THREADS; ++j) {
        const int idx = tid + THREADS * j;
        const int k = (split + (idx >> 7) * a.S) * TM + (idx & 127);
        vv[j] = (idx < nt * TM && k < na) ? a.active[(size_t)b * a.Kcap + k] : -1;
    }
#pragma unroll
    for (int j = 0; j < MAXT * TM / THREADS; ++j) {
        const int idx = tid + THREADS * j;
        if (idx < nt * TM) {
            ids_sh[idx] = vv[j];
            dts_sh[idx] = vv[j] >= 0 ? (float)(t_now - a.last_t[(size_t)b * a.V + vv[j]]) : 0.f;
        }
    }
    __syncthreads();

    auto issue_state = [&](int i) {
        if (i < nt) {
            unsigned char* dst = S_st + (i & 1) * STAGE_BYTES;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int idx = tid + THREADS * j, r = idx >> 4, c = idx & 15;
                const int v = ids_sh[i * TM + r];
                if (v >= 0) cp_async16(dst + r * 256 + ((c ^ (r & 15)) << 4), a.state + ((size_t)b * a.V + v) * N + c * 4);
            }
        }
        cp_commit();
    };
    auto issue_emb = [&](int i) {
        if (i < nt) {
            const __nv_bfloat16* E = (PASS == 1) ? a.Ek : a.Ev;
            unsigned char* dst = E_st + (i & 1) * STAGE_BYTES;
#pragma unroll
            for (int e = 0; e < HPC; ++e)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int idx = tid + THREADS * j, r = idx >> 3, c = idx & 7;
                    const int v = ids_sh[i * TM + r];
                    if (v >= 0) cp_async16(dst + e * ATOM_BYTES + r * 128 + ((c ^ (r & 7)) << 4), E + (size_t)v * D + (hp * HPC + e) * HD + c * 8);
                }
        }
        cp_commit();
    };
    issue_state(0);
    issue_emb(0);
    issue_state(1);
    issue_emb(1);
    {
        const float wscale = SILU ? 0.5f : 1.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int g = tid + THREADS * j, n = g >> 5, dd4 = (g & 31) * 4;
            // fp16 operands for the gate product (11 significant bits): state / 64 in the A tile, W * 64 here
            *reinterpret_cast<__half*>(B_sh + sw128_off(dd4 + 0, n)) = __float2half_rn(wv[j].x * wscale * STATE_F16_UNSCALE);
            *reinterpret_cast<__half*>(B_sh + sw128_off(dd4 + 1, n)) = __float2half_rn(wv[j].y * wscale * STATE_F16_UNSCALE);
            *reinterpret_cast<__half*>(B_sh + sw128_off(dd4 + 2, n)) = __float2half_rn(wv[j].z * wscale * STATE_F16_UNSCALE);
            *reinterpret_cast<__half*>(B_sh + sw128_off(dd4 + 3, n)) = __float2half_rn(wv[j].w * wscale * STATE_F16_UNSCALE);
        }
        if (PASS == 2)
            for (int i = tid; i < 1024; i += THREADS) reinterpret_cast<__nv_bfloat16*>(ones_sh)[i] = __float2bfloat16(1.0f);
        if (tid < N) l2r_sh[tid] = log2f(a.rhos[tid]);
        if (tid < ACC_COLS) q_sh[tid] = ld_dyn_f32(a.q, a.q_dt, ((size_t)b * a.H + hp * HPC) * HD + tid) * 0.125f;
    }
    // state stage -> decayed bf16 A tile; this thread: row `row`, channels [16 cg, 16 cg + 16)
    auto convert = [&](int i) {
        const unsigned char* src = S_st + (i & 1) * STAGE_BYTES + row * 256;
        const bool ok = ids_sh[i * TM + row] >= 0;
        const float dt = dts_sh[i * TM + row];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
            uint4 pk = make_uint4(0u, 0u, 0u, 0u);
            if (ok) {
                const int c0 = 4 * cg + 2 * cc;
                const float4 s0 = *reinterpret_cast<const float4*>(src + ((c0 ^ (row & 15)) << 4));
                const float4 s1 = *reinterpret_cast<const float4*>(src + (((c0 + 1) ^ (row & 15)) << 4));
                const float* lr = l2r_sh + 16 * cg + cc * 8;
                // state / 64 (STATE_F16_SCALE) folded into the exponent: 2^(dt log2 rho - 6)
                pk.x = pack_f16x2(s0.x * ex2_approx(fmaf(dt, lr[0], -6.0f)), s0.y * ex2_approx(fmaf(dt, lr[1], -6.0f)));
                pk.y = pack_f16x2(s0.z * ex2_approx(fmaf(dt, lr[2], -6.0f)), s0.w * ex2_approx(fmaf(dt, lr[3], -6.0f)));
                pk.z = pack_f16x2(s1.x * ex2_approx(fmaf(dt, lr[4], -6.0f)), s1.y * ex2_approx(fmaf(dt, lr[5], -6.0f)));
                pk.w = pack_f16x2(s1.z * ex2_approx(fmaf(dt, lr[6], -6.0f)), s1.w * ex2_approx(fmaf(dt, lr[7], -6.0f)));
            }
            *reinterpret_cast<uint4*>(A_sh + row * 128 + (((2 * cg + cc) ^ (row & 7)) << 4)) = pk;
        }
    };
    const uint32_t idesc = umma_idesc_16(TM, ACC_COLS, 0, 0, 0, 0);      // fp16 state tile, fp16 W
    const uint64_t da = umma_desc_k_sw128(smem_u32(A_sh)), db = umma_desc_k_sw128(smem_u32(B_sh));
    auto issue_gate = [&](uint32_t tmem_base, int i) {
#pragma unroll
        for (int k16 = 0; k16 < 4; ++k16)
            umma_bf16_ss(tmem_base + (uint32_t)((i & 1) * ACC_COLS), da + (uint64_t)((k16 * 32) >> 4), db + (uint64_t)((k16 * 32) >> 4), idesc, k16 != 0 ? 1u : 0u);
        umma_commit(&bars->acc_full[i & 1]);
    };

    cp_wait<3>();                                               // state stage of tile 0 landed (this thread's copies)
    __syncthreads();                                            // ... everyone's; B tile, q, barriers and TMEM address too
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;
    convert(0);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (tid == 0 && !bars->abort_flag) issue_gate(tmem_base, 0);
    issue_state(2);

    for (int i = 0; i < nt; ++i) {
        float prob = 0.f;                                       // fetched before the conversion work below, used after it
        if (PASS == 2 && ids_sh[i * TM + row] >= 0) prob = a.scores[((size_t)b * a.H + h) * a.Kcap + (split + i * a.S) * TM + row];
        cp_wait<2>();                                           // state stage of tile i+1 and embedding stage of tile i
        __syncthreads();
        if (!bars->abort_flag) mbar_wait(&bars->acc_full[i & 1], (uint32_t)((i >> 1) & 1), abort_flag);   // A tile free, accumulators of tile i ready
        tc_fence_after_sync();
        if (i + 1 < nt) {
            convert(i + 1);
            fence_proxy_async_smem();
            tc_fence_before_sync();
            __syncthreads();
            tc_fence_after_sync();
            if (tid == 0 && !bars->abort_flag) issue_gate(tmem_base, i + 1);
        }
        issue_state(i + 3);

        const bool ok = ids_sh[i * TM + row] >= 0;
        const uint32_t t_acc = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)((i & 1) * ACC_COLS + hh * HD + half * 32);
        const unsigned char* erow = E_st + (i & 1) * STAGE_BYTES + hh * ATOM_BYTES + row * 128;
        const float* qh = q_sh + hh * HD + half * 32;
        const int k = (split + i * a.S) * TM + row;
        if (PASS == 1) {
            float sp[2] = {0.f, 0.f};
            {
                float pre[32];
                tmem_ld_32x32b_x32(t_acc, pre);
                tmem_wait_ld();
#pragma unroll
                for (int j8 = 0; j8 < 4; ++j8) {
                    const uint4 e = *reinterpret_cast<const uint4*>(erow + (((half * 4 + j8) ^ (row & 7)) << 4));
                    const uint32_t ew[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
                    for (int pr = 0; pr < 4; ++pr) {
                        const int j = j8 * 8 + pr * 2;
                        const float h0 = pre[j], h1 = pre[j + 1];
                        const float g0 = SILU ? fmaf(h0, tanh_approx(h0), h0) : h0;
                        const float g1 = SILU ? fmaf(h1, tanh_approx(h1), h1) : h1;
                        sp[0] = fmaf(g0 * qh[j], bf16_lo(ew[pr]), sp[0]);
                        sp[1] = fmaf(g1 * qh[j + 1], bf16_hi(ew[pr]), sp[1]);
                    }
                }
            }
            // the two 32-column halves of a head add into a zeroed score: two addends, so the sum is order-independent
            if (ok) atomicAdd(a.scores + ((size_t)b * a.H + h) * a.Kcap + k, sp[0] + sp[1]);
            tc_fence_before_sync();
            __syncthreads();                                    // embedding stage i & 1 is free again
        } else {
            if (i > 0 && !bars->abort_flag) mbar_wait(&bars->pv_done, (uint32_t)((i - 1) & 1), abort_flag);   // V tile free
            unsigned char* vrow = V_sh + hh * ATOM_BYTES + row * 128;
            {
                float pre[32];
                tmem_ld_32x32b_x32(t_acc, pre);
                tmem_wait_ld();
#pragma unroll
                for (int j8 = 0; j8 < 4; ++j8) {
                    const uint4 e = *reinterpret_cast<const uint4*>(erow + (((half * 4 + j8) ^ (row & 7)) << 4));
                    const uint32_t ew[4] = {e.x, e.y, e.z, e.w};
                    uint32_t w[4];
#pragma unroll
                    for (int pr = 0; pr < 4; ++pr) {
                        const int j = j8 * 8 + pr * 2;
                        const float h0 = pre[j], h1 = pre[j + 1];
                        const float g0 = SILU ? fmaf(h0, tanh_approx(h0), h0) : h0;
                        const float g1 = SILU ? fmaf(h1, tanh_approx(h1), h1) : h1;
                        w[pr] = ok ? mul_bf16x2(pack_bf16x2(prob * g0, prob * g1), ew[pr]) : 0u;
                    }
                    st_shared_v4(vrow + (((half * 4 + j8) ^ (row & 7)) << 4), w[0], w[1], w[2], w[3]);
                }
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            __syncthreads();                // accumulators and embedding stage read, V tile written, by every warp
            tc_fence_after_sync();
            if (tid == 0 && !bars->abort_flag) {
                const uint32_t idesc2 = umma_idesc_bf16(ACC_COLS, 16, 1, 0);
                const uint64_t dv = umma_desc_mn_sw128(smem_u32(V_sh), ATOM_BYTES, 1024), d1 = umma_desc_k_sw128(smem_u32(ones_sh));
#pragma unroll
                for (int ks = 0; ks < TM / 16; ++ks)
                    umma_bf16_ss(tmem_base + 2 * ACC_COLS, dv + (uint64_t)(ks * (2048 >> 4)), d1, idesc2, (i != 0 || ks != 0) ? 1u : 0u);
                umma_commit(&bars->pv_done);
            }
        }
        issue_emb(i + 2);
    }
    cp_wait<0>();
    if (PASS == 2) {
        if (!bars->abort_flag) mbar_wait(&bars->pv_done, (uint32_t)((nt - 1) & 1), abort_flag);
        tc_fence_after_sync();
        if (cg == 0) {                      // lane = output column d of the head pair
            uint32_t r;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(tmem_base + 2 * ACC_COLS + ((uint32_t)((warp & 3) * 32) << 16)) : "memory");
            tmem_wait_ld();
            atomicAdd(a.O + ((size_t)b * a.H + hp * HPC) * HD + row, __uint_as_float(r));
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
    if (tid == 0 && bars->abort_flag) atomicOr(status, bars->abort_flag);   // sticky: never cleared by the library
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
                                      int flags, const int32_t* t_now_dev, void* workspace, size_t workspace_bytes,
                                      void* stream) {
    if (B < 0 || H < 1 || V < 1 || N < 1 || Kcap < 1) return MBEMA_ERR_SHAPE;
    if (hd != 64 || N != 64 || (H % 2) != 0 || B > 65535 || H > 65535) return MBEMA_ERR_UNSUPPORTED;
    if (B == 0) return MBEMA_OK;
    if (!q || !E_k || !E_v || !W_pe || !rhos || !state || !last_t || !active || !n_active || !O || !workspace) return MBEMA_ERR_NULL;
    if ((q_dtype != MBEMA_F32 && q_dtype != MBEMA_BF16) || (e_dtype != MBEMA_F32 && e_dtype != MBEMA_BF16)) return MBEMA_ERR_DTYPE;
    if (e_dtype != MBEMA_BF16) return MBEMA_ERR_UNSUPPORTED;     // rows are copied as stored into the bf16 operand rings
    if (((uintptr_t)E_k | (uintptr_t)E_v | (uintptr_t)state) & 15) return MBEMA_ERR_ALIGN;
    if (workspace_bytes < mbema_decode_attend_tc_workspace_bytes(B, H, Kcap)) return MBEMA_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    int* status = reinterpret_cast<int*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
    // CTAs per (sequence, head pair)
    const int ntiles = (int)((Kcap + dtc::TM - 1) / dtc::TM);
    int sm_count = 148;
    {
        int dev = 0;
        MBEMA_CUDA_TRY(cudaGetDevice(&dev));
        MBEMA_CUDA_TRY(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
    }
    // every CTA costs about 1.5 tile times of setup and the grid runs in waves of one CTA per SM: pick the split
    // with the fewest (waves x (tiles per CTA + setup)), at most MAXT tiles per CTA
    int64_t S = ntiles;
    {
        const int64_t groups = B * (H / 2), s_min = (ntiles + dtc::MAXT - 1) / dtc::MAXT;
        double best = 1e30;
        for (int64_t c = s_min; c <= ntiles; ++c) {
            const int64_t waves = (groups * c + sm_count - 1) / sm_count, per = (ntiles + c - 1) / c;
            const double cost = (double)waves * ((double)per + 1.5);
            if (cost < best) { best = cost; S = c; }
        }
    }
    if (S > 65535) return MBEMA_ERR_UNSUPPORTED;
    dtc::Args a{q, q_dtype, reinterpret_cast<const __nv_bfloat16*>(E_k), reinterpret_cast<const __nv_bfloat16*>(E_v), W_pe, rhos,
                state, last_t, active, n_active, reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(status) + 256), O,
                (int)B, (int)H, (int)V, (int)Kcap, (int)t_now, (int)S, t_now_dev, (float)V_total,
                (flags & MBEMA_FLAG_LISTED_ONLY) ? 1 : 0};
    MBEMA_CUDA_TRY(cudaMemsetAsync(O, 0, (size_t)B * H * hd * sizeof(float), st));
    MBEMA_CUDA_TRY(cudaMemsetAsync(a.scores, 0, (size_t)B * H * Kcap * sizeof(float), st));
    const int smem = dtc::SMEM_BYTES;
    dim3 grid((unsigned)S, (unsigned)(H / 2), (unsigned)B);
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
