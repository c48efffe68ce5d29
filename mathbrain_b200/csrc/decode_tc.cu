// Streaming decode on the tensor cores (MBEMA_MODE_TC_BF16, N = 64, bf16 slot embeddings): attention of ONE query
// per sequence over the slots seen so far, in ONE walk over the slots.  Rows of a tile are SLOTS here (a thread per
// slot and 32-column half of a head), so the softmax runs across threads:
//   per 128-slot tile   decayed state tile (fp16) -> tcgen05.mma against W -> gate -> score s[k] per head (the two
//                       halves of a head meet in shared memory) -> tile maximum m -> p = exp(s - m) ->
//                       the bf16 tile (p * gate * E_v)[k, d] is summed over its 128 slots by a second tcgen05.mma
//                       against a ones operand (the column-sum trick of the training backward) into a fresh TMEM
//                       region, which the CTA folds into its running (max, normaliser, output) one tile later;
//   per CTA             partial (m, l, O[128]) of its tiles, written to the workspace;
//   merge kernel        per (sequence, head): the partials of all CTAs plus the mass of the never-seen slots
//                       (exp(0 - m) each) -> O.
// The gate product, its tanh and every gather are done once per slot and head pair.  Embedding rows are cp.async
// copies two tiles ahead into shared-memory rings; state rows are prefetched into registers a tile ahead (64 bytes a
// thread), so the tile of slot tile i+1 is converted and its UMMA issued before the epilogue of tile i.
#include "common.cuh"
#include <cuda_fp16.h>
#include "sm100_ptx.cuh"

#include <algorithm>
namespace mbema {
namespace dtc {

using namespace ptx;

static constexpr int TM = 128, HD = 64, HPC = 2, N = 64, ACC_COLS = HPC * HD, THREADS = 512, MAXT = 16;
static constexpr int ATOM_BYTES = TM * 128;
static constexpr int STAGE_BYTES = 2 * ATOM_BYTES;            // one embedding stage: 2 heads x 128 rows x 128 B
static constexpr int PART_FLOATS = ACC_COLS + 4;              // per-CTA partial: O[128], m[2], l[2]
static constexpr int OFF_B = 0, OFF_A = ATOM_BYTES, OFF_EK = 2 * ATOM_BYTES, OFF_EV = OFF_EK + 2 * STAGE_BYTES,
                     OFF_V = OFF_EV + 2 * STAGE_BYTES, OFF_ONES = OFF_V + 2 * ATOM_BYTES, OFF_Q = OFF_ONES + 2048,
                     OFF_L2R = OFF_Q + 512, OFF_IDS = OFF_L2R + 256, OFF_DTS = OFF_IDS + MAXT * TM * 4,
                     OFF_SC = OFF_DTS + MAXT * TM * 4, OFF_WRED = OFF_SC + TM * 4 * 4, OFF_TILE = OFF_WRED + 2 * 16 * 4,
                     OFF_BARS = OFF_TILE + MAXT * 4 * 4, SMEM_BYTES = OFF_BARS + 64 + 1024;
static constexpr int COL_R = 2 * ACC_COLS;                    // TMEM: two gate accumulators, then two 16-column sum regions

struct Args {
    const void* q; int q_dt;
    const __nv_bfloat16* Ek; const __nv_bfloat16* Ev;
    const float* W; const float* rhos;
    const float* state; const int* last_t; const int* active; const int* n_active;
    float* part;                   // [B, H/2, S, PART_FLOATS]: per-CTA partial results
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
__device__ __forceinline__ float tmem_ld_1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    return __uint_as_float(r);
}

struct Bars { uint64_t acc_full[2]; uint64_t pv_done[2]; uint32_t tmem_base; int abort_flag; };

template <bool SILU>
__global__ void __launch_bounds__(THREADS, 1) k_decode_tc(Args a, int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* A_sh = sm + OFF_A;
    unsigned char* B_sh = sm + OFF_B;
    unsigned char* Ek_st = sm + OFF_EK;     // [2 stages][head][128 rows][8 chunks of 8 bf16, chunk ^ (row & 7)]
    unsigned char* Ev_st = sm + OFF_EV;
    unsigned char* V_sh = sm + OFF_V;       // [head][128 k][64 d] bf16, MN-major operand of the column sum
    unsigned char* ones_sh = sm + OFF_ONES;
    float* q_sh = reinterpret_cast<float*>(sm + OFF_Q);                 // q / sqrt(hd) of the two heads
    float* l2r_sh = reinterpret_cast<float*>(sm + OFF_L2R);
    int* ids_sh = reinterpret_cast<int*>(sm + OFF_IDS);                 // slot of every row of this CTA's tiles, -1 = none
    float* dts_sh = reinterpret_cast<float*>(sm + OFF_DTS);             // steps since that slot's last update
    float* sc_sh = reinterpret_cast<float*>(sm + OFF_SC);               // [128 rows][4 column groups] partial scores
    float* wmax_sh = reinterpret_cast<float*>(sm + OFF_WRED);           // [16 warps] maxima, then [16 warps] sums of p
    float* wsum_sh = wmax_sh + 16;
    float* tile_sh = reinterpret_cast<float*>(sm + OFF_TILE);           // [tile][head] maximum, [tile][2 + head] sum of p
    Bars* bars = reinterpret_cast<Bars*>(sm + OFF_BARS);
    volatile int* abort_flag = &bars->abort_flag;

    const int split = blockIdx.x, hp = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cg = tid >> 7, row = tid & 127;                   // column group: head cg >> 1 of the pair, 32-column half cg & 1
    const int hh = cg >> 1, half = cg & 1;
    const int D = a.H * HD;
    const int na = min(a.n_active[b], a.Kcap);
    const int ntile_b = (na + TM - 1) / TM;
    if (split >= ntile_b) return;                               // uniform per CTA
    const int nt = min((ntile_b - split + a.S - 1) / a.S, MAXT);

    if (tid == 0) {
        mbar_init(&bars->acc_full[0], 1);
        mbar_init(&bars->acc_full[1], 1);
        mbar_init(&bars->pv_done[0], 1);
        mbar_init(&bars->pv_done[1], 1);
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

    // state row of this thread's slot in tile i, channels [16 cg, 16 cg + 16), straight into registers
    float4 sreg[4];
    auto load_state = [&](int i) {
        const int v = i < nt ? ids_sh[i * TM + row] : -1;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            sreg[j] = v >= 0 ? __ldg(reinterpret_cast<const float4*>(a.state + ((size_t)b * a.V + v) * N + 16 * cg + 4 * j))
                             : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto issue_emb = [&](int i) {
        if (i < nt) {
#pragma unroll
            for (int kv = 0; kv < 2; ++kv) {
                const __nv_bfloat16* E = kv == 0 ? a.Ek : a.Ev;
                unsigned char* dst = (kv == 0 ? Ek_st : Ev_st) + (i & 1) * STAGE_BYTES;
#pragma unroll
                for (int e = 0; e < HPC; ++e)
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int idx = tid + THREADS * j, r = idx >> 3, c = idx & 7;
                        const int v = ids_sh[i * TM + r];
                        if (v >= 0) cp_async16(dst + e * ATOM_BYTES + r * 128 + ((c ^ (r & 7)) << 4), E + (size_t)v * D + (hp * HPC + e) * HD + c * 8);
                    }
            }
        }
        cp_commit();
    };
    load_state(0);
    issue_emb(0);
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
        for (int i = tid; i < 1024; i += THREADS) reinterpret_cast<__nv_bfloat16*>(ones_sh)[i] = __float2bfloat16(1.0f);
        if (tid < N) l2r_sh[tid] = log2f(a.rhos[tid]);
        if (tid < ACC_COLS) q_sh[tid] = ld_dyn_f32(a.q, a.q_dt, ((size_t)b * a.H + hp * HPC) * HD + tid) * 0.125f;
    }
    // prefetched state registers -> decayed fp16 A tile; this thread: row `row`, channels [16 cg, 16 cg + 16)
    auto convert = [&](int i) {
        const bool ok = ids_sh[i * TM + row] >= 0;
        const float dt = dts_sh[i * TM + row];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
            uint4 pk = make_uint4(0u, 0u, 0u, 0u);
            if (ok) {
                const float4 s0 = sreg[2 * cc], s1 = sreg[2 * cc + 1];
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

    __syncthreads();                                            // B tile, q, ones, barriers and the TMEM address
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;
    convert(0);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (tid == 0 && !bars->abort_flag) issue_gate(tmem_base, 0);
    load_state(1);

    // running softmax state of output column `row` of the head pair (threads of column group 0), head row >> 6
    float m_run = -INFINITY, l_run = 0.f, o_run = 0.f;
    const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    auto fold = [&](int j) {        // tile j's column sums (its PV product has completed) into the running state
        const float mt = tile_sh[j * 4 + (row >> 6)], lt = tile_sh[j * 4 + 2 + (row >> 6)];
        const float v = tmem_ld_1(t_lane + (uint32_t)(COL_R + (j & 1) * 16));
        tmem_wait_ld();
        const float m_new = fmaxf(m_run, mt);
        const float c_old = __expf(m_run - m_new), c_new = __expf(mt - m_new);     // exp(-inf) = 0 on the first tile
        o_run = o_run * c_old + v * c_new;
        l_run = l_run * c_old + lt * c_new;
        m_run = m_new;
    };

    for (int i = 0; i < nt; ++i) {
        if (!bars->abort_flag) mbar_wait(&bars->acc_full[i & 1], (uint32_t)((i >> 1) & 1), abort_flag);   // A tile free, accumulators of tile i ready
        tc_fence_after_sync();
        if (i + 1 < nt) {
            convert(i + 1);
            fence_proxy_async_smem();
            tc_fence_before_sync();
        }
        cp_wait<1>();                                           // embedding stages of tile i (this thread's copies)
        __syncthreads();                                        // ... everyone's, and the whole A tile of tile i + 1
        tc_fence_after_sync();
        if (i + 1 < nt && tid == 0 && !bars->abort_flag) issue_gate(tmem_base, i + 1);
        load_state(i + 2);

        const bool ok = ids_sh[i * TM + row] >= 0;
        const uint32_t t_acc = t_lane + (uint32_t)((i & 1) * ACC_COLS + hh * HD + half * 32);
        const unsigned char* ekrow = Ek_st + (i & 1) * STAGE_BYTES + hh * ATOM_BYTES + row * 128;
        const unsigned char* evrow = Ev_st + (i & 1) * STAGE_BYTES + hh * ATOM_BYTES + row * 128;
        const float* qh = q_sh + hh * HD + half * 32;
        // ---- gate of this thread's 32 columns (kept) and its part of the score
        float g[32];
        float sp[2] = {0.f, 0.f};
        {
            float pre[32];
            tmem_ld_32x32b_x32(t_acc, pre);
            tmem_wait_ld();
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
                const uint4 e = *reinterpret_cast<const uint4*>(ekrow + (((half * 4 + j8) ^ (row & 7)) << 4));
                const uint32_t ew[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
                for (int pr = 0; pr < 4; ++pr) {
                    const int j = j8 * 8 + pr * 2;
                    const float h0 = pre[j], h1 = pre[j + 1];
                    g[j] = SILU ? fmaf(h0, tanh_approx(h0), h0) : h0;
                    g[j + 1] = SILU ? fmaf(h1, tanh_approx(h1), h1) : h1;
                    sp[0] = fmaf(g[j] * qh[j], bf16_lo(ew[pr]), sp[0]);
                    sp[1] = fmaf(g[j + 1] * qh[j + 1], bf16_hi(ew[pr]), sp[1]);
                }
            }
        }
        sc_sh[row * 4 + cg] = sp[0] + sp[1];
        tc_fence_before_sync();
        __syncthreads();                                        // both halves of every score; accumulators of tile i read
        const float s = ok ? sc_sh[row * 4 + 2 * hh] + sc_sh[row * 4 + 2 * hh + 1] : -INFINITY;
        {
            float mx = s;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            if (lane == 0) wmax_sh[warp] = mx;
        }
        __syncthreads();
        const float mt = fmaxf(fmaxf(wmax_sh[8 * hh], wmax_sh[8 * hh + 1]), fmaxf(wmax_sh[8 * hh + 2], wmax_sh[8 * hh + 3]));
        const float prob = ok ? __expf(s - mt) : 0.f;            // every tile holds at least one slot, so mt is finite
        if (half == 0) {
            const float ps = warp_sum(prob);
            if (lane == 0) wsum_sh[warp] = ps;
        }
        // ---- V tile: (p * gate * E_v)[k, d] in bf16; the column sum of tile i - 2 used the other TMEM region, the V tile
        // itself was last read by the product of tile i - 1
        if (i > 0 && !bars->abort_flag) mbar_wait(&bars->pv_done[(i - 1) & 1], (uint32_t)(((i - 1) >> 1) & 1), abort_flag);
        tc_fence_after_sync();
        {
            unsigned char* vrow = V_sh + hh * ATOM_BYTES + row * 128;
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
                const uint4 e = *reinterpret_cast<const uint4*>(evrow + (((half * 4 + j8) ^ (row & 7)) << 4));
                const uint32_t ew[4] = {e.x, e.y, e.z, e.w};
                uint32_t w[4];
#pragma unroll
                for (int pr = 0; pr < 4; ++pr) {
                    const int j = j8 * 8 + pr * 2;
                    w[pr] = ok ? mul_bf16x2(pack_bf16x2(prob * g[j], prob * g[j + 1]), ew[pr]) : 0u;
                }
                st_shared_v4(vrow + (((half * 4 + j8) ^ (row & 7)) << 4), w[0], w[1], w[2], w[3]);
            }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();                // V tile written, embedding stages read, per-warp sums of p stored, by every warp
        tc_fence_after_sync();
        if (tid == 0 && !bars->abort_flag) {
            const uint32_t idesc2 = umma_idesc_bf16(ACC_COLS, 16, 1, 0);
            const uint64_t dv = umma_desc_mn_sw128(smem_u32(V_sh), ATOM_BYTES, 1024), d1 = umma_desc_k_sw128(smem_u32(ones_sh));
#pragma unroll
            for (int ks = 0; ks < TM / 16; ++ks)
                umma_bf16_ss(tmem_base + (uint32_t)(COL_R + (i & 1) * 16), dv + (uint64_t)(ks * (2048 >> 4)), d1, idesc2, ks != 0 ? 1u : 0u);
            umma_commit(&bars->pv_done[i & 1]);
        }
        if (tid < 2) {                  // head `tid`: this tile's maximum and sum of p (column-group 2 tid holds half 0)
            tile_sh[i * 4 + tid] = fmaxf(fmaxf(wmax_sh[8 * tid], wmax_sh[8 * tid + 1]), fmaxf(wmax_sh[8 * tid + 2], wmax_sh[8 * tid + 3]));
            tile_sh[i * 4 + 2 + tid] = wsum_sh[8 * tid] + wsum_sh[8 * tid + 1] + wsum_sh[8 * tid + 2] + wsum_sh[8 * tid + 3];
        }
        if (i > 0 && cg == 0) fold(i - 1);      // its product completed (waited for above); tile_sh[i - 1] was written an iteration ago
        issue_emb(i + 2);
    }
    cp_wait<0>();
    if (!bars->abort_flag) mbar_wait(&bars->pv_done[(nt - 1) & 1], (uint32_t)(((nt - 1) >> 1) & 1), abort_flag);
    tc_fence_after_sync();
    __syncthreads();                                            // tile_sh of the last tile
    if (cg == 0) {
        fold(nt - 1);
        float* part = a.part + (((size_t)b * (a.H / HPC) + hp) * a.S + split) * PART_FLOATS;
        part[row] = o_run;
        if ((row & 63) == 0) {
            part[ACC_COLS + (row >> 6)] = m_run;
            part[ACC_COLS + 2 + (row >> 6)] = l_run;
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

// O[b, h, :] from the partials of the CTAs that walked sequence b: softmax over all V_total slots (the never-seen
// ones have score 0 and no value, they only add exp(0 - m) each to the normaliser)
__global__ void __launch_bounds__(HD) k_decode_merge(Args a) {
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const int na = min(a.n_active[b], a.Kcap);
    const int ntile_b = (na + TM - 1) / TM;
    const int ns = min(a.S, ntile_b);
    const float rest = a.listed_only ? 0.f : fmaxf(a.v_total - (float)na, 0.f);
    const float* part = a.part + ((size_t)b * (a.H / HPC) + h / HPC) * a.S * PART_FLOATS;
    const int hh = h % HPC;
    float m = rest > 0.f ? 0.f : -INFINITY;
    for (int s = 0; s < ns; ++s) m = fmaxf(m, part[(size_t)s * PART_FLOATS + ACC_COLS + hh]);
    float l = rest > 0.f ? rest * __expf(-m) : 0.f, o = 0.f;
    for (int s = 0; s < ns; ++s) {
        const float* p = part + (size_t)s * PART_FLOATS;
        const float c = __expf(p[ACC_COLS + hh] - m);
        l += p[ACC_COLS + 2 + hh] * c;
        o += p[hh * HD + d] * c;
    }
    a.O[((size_t)b * a.H + h) * HD + d] = l > 0.f ? o / l : 0.f;
}

}  // namespace dtc
}  // namespace mbema

using namespace mbema;

extern "C" size_t mbema_decode_attend_tc_workspace_bytes(int64_t B, int64_t H, int64_t Kcap) {
    const size_t ntiles = (size_t)((Kcap + dtc::TM - 1) / dtc::TM);       // at most one CTA per tile and head pair
    return 512 + (size_t)B * (size_t)(H / 2 > 0 ? H / 2 : 1) * ntiles * dtc::PART_FLOATS * sizeof(float);
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
    const int smem = dtc::SMEM_BYTES;
    dim3 grid((unsigned)S, (unsigned)(H / 2), (unsigned)B);
    const bool silu = (flags & MBEMA_FLAG_SILU) != 0;
#define MBEMA_DECODE_LAUNCH(S_)                                                                                     \
    do {                                                                                                           \
        MBEMA_CUDA_TRY(cudaFuncSetAttribute(dtc::k_decode_tc<S_>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
        dtc::k_decode_tc<S_><<<grid, dtc::THREADS, smem, st>>>(a, status);                                         \
    } while (0)
    if (silu) MBEMA_DECODE_LAUNCH(true); else MBEMA_DECODE_LAUNCH(false);
#undef MBEMA_DECODE_LAUNCH
    int rc = check_launch();
    if (rc) return rc;
    dtc::k_decode_merge<<<dim3((unsigned)H, (unsigned)B), dtc::HD, 0, st>>>(a);
    return check_launch();
}
