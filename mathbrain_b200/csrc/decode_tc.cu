// Streaming decode on the tensor cores (MBEMA_MODE_TC_BF16, N = 64, bf16 slot embeddings): attention of ONE query
// per sequence over the slots seen so far, in ONE walk over the slots, warp-specialised like the training kernels.
// A CTA owns (sequence, head pair, share of the 128-slot tiles); rows of a tile are SLOTS.
//   eight producer warps (two threads per slot): cp.async gathers of the tile's E_k / E_v rows into two-stage rings, the
//       slot's state row from global memory -> decayed fp16 row of the A tile.  A tile's stages are released piecewise:
//       the E_k rows, the A tile and the accumulators once the epilogue has finished its first pass over tile i - 2,
//       the E_v rows only when that tile's column sum has completed, so only the E_v copies wait for the later event;
//   one issuing warp (one lane): every tcgen05.mma of the CTA, gate products (against W, accumulators in TMEM, two
//       stages) and column sums, so that no producer thread ever waits for the epilogue's operand tile;
//   sixteen epilogue warps (a thread per slot and HALF a head, 32 columns): gate = SiLU of the accumulators, partial
//       score sum_c q g E_k in the thread; both halves post their partial sums in shared memory, the head's eight warps
//       meet on an mbarrier, and every warp forms the rows' scores and the head's tile maximum from the 128 posted
//       pairs; p = exp(s - m), the bf16 tile (p * gate * E_v)[k, d] written over the E_v rows it was made from; its
//       sum over the 128 slots is a second tcgen05.mma against a ones operand (the column-sum trick of the training
//       backward) into one of two TMEM regions, which warps 0..3 fold into the CTA's running (max, normaliser, output)
//       one tile later (online softmax in registers);
//   per CTA      partial (O[128], m[2], l[2]) of its tiles, written to the workspace;
//   merge kernel per (sequence, head): the partials of all CTAs plus the mass of the never-seen slots -> O.
// No block barrier inside the tile loop: the roles meet on mbarriers (every wait bounded), so the gathers, the state
// conversion and the gate product of tile i+1 run while the epilogue works on tile i.
#include "common.cuh"
#include <cuda_fp16.h>
#include "sm100_ptx.cuh"

#include <algorithm>
namespace mbema {
namespace dtc {

using namespace ptx;

static constexpr int TM = 128, HD = 64, HPC = 2, N = 64, ACC_COLS = HPC * HD, MAXT = 16;
static constexpr int EPI_WARPS = 16, PROD_WARPS = 8, MMA_WARP = EPI_WARPS + PROD_WARPS, THREADS = (MMA_WARP + 1) * 32;
static constexpr int HALF = HD / 2;                           // columns of a head per epilogue thread
static constexpr int ATOM_BYTES = TM * 128;
static constexpr int STAGE_BYTES = 2 * ATOM_BYTES;            // one embedding stage: 2 heads x 128 rows x 128 B
static constexpr int PART_FLOATS = ACC_COLS + 4;              // per-CTA partial: O[128], m[2], l[2]
static constexpr int OFF_B = 0, OFF_A = ATOM_BYTES, OFF_EK = OFF_A + 2 * ATOM_BYTES, OFF_EV = OFF_EK + 2 * STAGE_BYTES,
                     OFF_ONES = OFF_EV + 2 * STAGE_BYTES, OFF_Q = OFF_ONES + 2048, OFF_L2R = OFF_Q + 512,
                     OFF_IDS = OFF_L2R + 256, OFF_DTS = OFF_IDS + MAXT * TM * 4, OFF_WRED = OFF_DTS + MAXT * TM * 4,
                     OFF_XCH = OFF_WRED + 4 * 16 * 4, OFF_BARS = OFF_XCH + 2 * HPC * 2 * TM * 4, SMEM_BYTES = OFF_BARS + 192 + 1024;
static constexpr int COL_R = 2 * ACC_COLS;                    // TMEM: two gate accumulators, then two 16-column sum regions
// no setmaxnreg here: 800 threads at 80 registers; neither role needs more

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

struct Bars {
    uint64_t a_full[2];          // every producer warp has written its part of the A tile                 (8 arrivals)
    uint64_t acc_full[2];        // gate product done (1 commit) + every producer warp's E_k rows have landed (8 arrivals)
    uint64_t ev_full[2];         // every producer warp's E_v rows have landed                              (8 arrivals)
    uint64_t acc_empty[2];       // every epilogue warp has read the stage's accumulators                 (8 arrivals)
    uint64_t v_full[2];          // every epilogue warp has written its rows of the column-sum operand     (8 arrivals)
    uint64_t pv_done[2];         // column-sum product done: the E stages of that tile are free            (1 commit)
    uint64_t hbar[2];            // per head: its eight epilogue warps have posted their rows' partial scores (8 arrivals)
    uint64_t drain;              // the issuing lane's products have completed (teardown)                  (1 arrival)
    uint32_t tmem_base;
    int abort_flag;
    int drain_flag;
};
static_assert(sizeof(Bars) <= 192, "barrier block");

template <bool SILU>
__global__ void __launch_bounds__(THREADS, 1) k_decode_tc(Args a, int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* A_sh = sm + OFF_A;       // [2 stages][128 rows][64 channels] fp16, K-major, 128-byte swizzle
    unsigned char* B_sh = sm + OFF_B;
    unsigned char* Ek_st = sm + OFF_EK;     // [2 stages][head][128 rows][8 chunks of 8 bf16, chunk ^ (row & 7)]
    unsigned char* Ev_st = sm + OFF_EV;     // same; rewritten in place as (p * gate * E_v)[k, d], the MN-major operand of the column sum
    unsigned char* ones_sh = sm + OFF_ONES;
    float* q_sh = reinterpret_cast<float*>(sm + OFF_Q);                 // q / sqrt(hd) of the two heads
    float* l2r_sh = reinterpret_cast<float*>(sm + OFF_L2R);
    int* ids_sh = reinterpret_cast<int*>(sm + OFF_IDS);                 // slot of every row of this CTA's tiles, -1 = none
    float* dts_sh = reinterpret_cast<float*>(sm + OFF_DTS);             // steps since that slot's last update
    float* wred = reinterpret_cast<float*>(sm + OFF_WRED);              // [tile & 3][16]: tile maximum per head at 0..1, sums of p per (head, warp of its first half) at 4..11
    float* xch = reinterpret_cast<float*>(sm + OFF_XCH);                // [tile & 1][head][half][128 rows]: partial scores
    Bars* bars = reinterpret_cast<Bars*>(sm + OFF_BARS);
    volatile int* abort_flag = &bars->abort_flag;

    const int split = blockIdx.x, hp = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = (warp & 3) * 32 + lane;                     // slot within the tile (== TMEM lane of the epilogue warps)
    const bool is_epi = warp < EPI_WARPS;
    const int D = a.H * HD;
    const int na = min(a.n_active[b], a.Kcap);
    const int ntile_b = (na + TM - 1) / TM;
    if (split >= ntile_b) return;                               // uniform per CTA
    const int nt = min((ntile_b - split + a.S - 1) / a.S, MAXT);

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->a_full[i], PROD_WARPS);
            mbar_init(&bars->acc_full[i], 1 + PROD_WARPS);
            mbar_init(&bars->ev_full[i], PROD_WARPS);
            mbar_init(&bars->acc_empty[i], EPI_WARPS);
            mbar_init(&bars->v_full[i], EPI_WARPS);
            mbar_init(&bars->pv_done[i], 1);
        }
        mbar_init(&bars->hbar[0], 8);
        mbar_init(&bars->hbar[1], 8);
        mbar_init(&bars->drain, 1);
        bars->drain_flag = 0;
        bars->abort_flag = *reinterpret_cast<volatile int*>(status);
        fence_barrier_init();
    }
    if (warp == EPI_WARPS) {
        tmem_alloc(&bars->tmem_base, 512);
        tmem_relinquish();
    }
    // producer threads (two per slot of a tile): slot prow, channels [32 phalf, 32 phalf + 32); 16-byte chunk c of four rows' E rows
    const bool is_prod = !is_epi && warp != MMA_WARP;
    const int ptid = tid - EPI_WARPS * 32;
    const int prow = ptid & 127, phalf = (ptid >> 7) & 1;
    const int c = ptid & 7;
    float4 sr[8];        // a producer thread's half of its slot's state row, all of it in flight at once, one tile ahead of its use
    auto load_state = [&](int i) {
        const int v = i < nt ? ids_sh[i * TM + prow] : -1;
        const float4* src = reinterpret_cast<const float4*>(a.state + ((size_t)b * a.V + (v >= 0 ? v : 0)) * N + 32 * phalf);
#pragma unroll
        for (int j = 0; j < 8; ++j) sr[j] = v >= 0 ? __ldg(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    // this thread's 8 copies of 16 bytes of tile i's E_k (or E_v) rows, both heads, into the tile's stage
    auto issue_rows = [&](unsigned char* stage0, const __nv_bfloat16* table, int i, const int (&vj)[4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = (ptid + PROD_WARPS * 32 * j) >> 3;
            if (vj[j] >= 0) {
                const size_t src = (size_t)vj[j] * D + hp * ACC_COLS + c * 8;
                const int dst = (i & 1) * STAGE_BYTES + r * 128 + ((c ^ (r & 7)) << 4);
                cp_async16(stage0 + dst, table + src);
                cp_async16(stage0 + dst + ATOM_BYTES, table + src + HD);
            }
        }
    };
    {   // this CTA's slots and their ages, and the operands every tile shares: W (fp16, times 64; times 1/2 for SiLU), ones,
        // decay logs, q.  The slot ids are fetched first and the ages (a dependent load) after the W block, so that the
        // two round trips to memory run under the W loads instead of after them: a CTA walks only a few tiles and the time
        // to its first one counts.
        constexpr int IDS_PER_THREAD = (MAXT * TM + THREADS - 1) / THREADS;
        int vs[IDS_PER_THREAD];
#pragma unroll
        for (int j = 0; j < IDS_PER_THREAD; ++j) {
            const int idx = tid + j * THREADS;
            const int k = (split + (idx >> 7) * a.S) * TM + (idx & 127);
            vs[j] = (idx < nt * TM && k < na) ? __ldg(a.active + (size_t)b * a.Kcap + k) : -1;
        }
        const int t_now = a.t_dev ? *a.t_dev : a.t_now;
#pragma unroll
        for (int j = 0; j < IDS_PER_THREAD; ++j) {
            const int idx = tid + j * THREADS;
            if (idx < nt * TM) ids_sh[idx] = vs[j];
        }
        __syncthreads();
        // the producers' fetches for the first tile start here, under the W loads and the second round trip (the ages)
        if (is_prod) {
            int vj[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) vj[j] = ids_sh[(ptid + PROD_WARPS * 32 * j) >> 3];
            issue_rows(Ek_st, a.Ek, 0, vj);
            cp_commit();                 // group E_k(0)
            issue_rows(Ev_st, a.Ev, 0, vj);
            cp_commit();                 // group E_v(0)
            load_state(0);
        }
        const float wscale = (SILU ? 0.5f : 1.0f) * STATE_F16_UNSCALE;
        for (int idx = tid; idx < N * ACC_COLS / 4; idx += THREADS) {
            const int n = idx >> 5, dd4 = (idx & 31) * 4;
            const float4 w = __ldg(reinterpret_cast<const float4*>(a.W + (size_t)n * D + hp * ACC_COLS + dd4));
            *reinterpret_cast<__half*>(B_sh + sw128_off(dd4 + 0, n)) = __float2half_rn(w.x * wscale);
            *reinterpret_cast<__half*>(B_sh + sw128_off(dd4 + 1, n)) = __float2half_rn(w.y * wscale);
            *reinterpret_cast<__half*>(B_sh + sw128_off(dd4 + 2, n)) = __float2half_rn(w.z * wscale);
            *reinterpret_cast<__half*>(B_sh + sw128_off(dd4 + 3, n)) = __float2half_rn(w.w * wscale);
        }
        int lt[IDS_PER_THREAD];
#pragma unroll
        for (int j = 0; j < IDS_PER_THREAD; ++j) lt[j] = vs[j] >= 0 ? a.last_t[(size_t)b * a.V + vs[j]] : 0;
        for (int i = tid; i < 1024; i += THREADS) reinterpret_cast<__nv_bfloat16*>(ones_sh)[i] = __float2bfloat16(1.0f);
        if (tid < N) l2r_sh[tid] = log2f(a.rhos[tid]);
        if (tid < ACC_COLS) q_sh[tid] = ld_dyn_f32(a.q, a.q_dt, ((size_t)b * a.H + hp * HPC) * HD + tid) * 0.125f;
#pragma unroll
        for (int j = 0; j < IDS_PER_THREAD; ++j) {
            const int idx = tid + j * THREADS;
            if (idx < nt * TM) dts_sh[idx] = vs[j] >= 0 ? (float)(t_now - lt[j]) : 0.f;
        }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;

    if (warp == MMA_WARP) {
        // ============================================================ issuing warp: one lane issues every tcgen05.mma of the CTA
        // A warp of its own, so that no producer thread ever waits for the epilogue's operand tile: in order
        // gate(0), gate(1), sum(0), gate(2), sum(1), ...
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_16(TM, ACC_COLS, 0, 0, 0, 0);      // fp16 state tile, fp16 W
            const uint32_t idesc2 = umma_idesc_bf16(ACC_COLS, 16, 1, 0);         // column sum: A = tile (MN-major), B = ones
            const uint64_t db = umma_desc_k_sw128(smem_u32(B_sh)), d1 = umma_desc_k_sw128(smem_u32(ones_sh));
            auto issue_pv = [&](int j) -> bool {        // column sums of tile j, once the epilogue has written the operand
                if (!mbar_wait(&bars->v_full[j & 1], (uint32_t)((j >> 1) & 1), abort_flag, 5)) return false;
                tc_fence_after_sync();
                const uint64_t dv = umma_desc_mn_sw128(smem_u32(Ev_st + (j & 1) * STAGE_BYTES), ATOM_BYTES, 1024);
#pragma unroll
                for (int ks = 0; ks < TM / 16; ++ks)
                    umma_bf16_ss(tmem_base + (uint32_t)(COL_R + (j & 1) * 16), dv + (uint64_t)(ks * (2048 >> 4)), d1, idesc2, ks != 0 ? 1u : 0u);
                umma_commit(&bars->pv_done[j & 1]);
                return true;
            };
            bool go = true;
            for (int i = 0; i < nt && go; ++i) {
                const int st = i & 1, u = i >> 1;
                go = mbar_wait(&bars->a_full[st], (uint32_t)(u & 1), abort_flag, 3);
                if (go && i >= 2) go = mbar_wait(&bars->acc_empty[st], (uint32_t)((u - 1) & 1), abort_flag, 4);
                if (go) {
                    tc_fence_after_sync();
                    const uint64_t da = umma_desc_k_sw128(smem_u32(A_sh + st * ATOM_BYTES));
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16)
                        umma_bf16_ss(tmem_base + (uint32_t)(st * ACC_COLS), da + (uint64_t)((k16 * 32) >> 4), db + (uint64_t)((k16 * 32) >> 4), idesc, k16 != 0 ? 1u : 0u);
                    umma_commit(&bars->acc_full[st]);
                    if (i >= 1) go = issue_pv(i - 1);
                }
            }
            if (go && nt > 0) issue_pv(nt - 1);
            umma_commit(&bars->drain);       // arrives once every product issued above has completed
        }
    } else if (!is_epi) {
        // ============================================================ producer warps: two threads per slot of the tile
        // (the copies and the state row of tile 0 were issued in the prologue)
        int done = 0;                    // tiles whose E_v copies this thread has issued
        for (int i = 0; i < nt; ++i) {
            const int st = i & 1, u = i >> 1;
            // The tile's stages are released piecewise.  The E_k rows and the accumulators of tile i - 2 are free once the
            // epilogue has finished its first pass over them (its A tile even earlier: the gate product has completed);
            // the E_v rows only once that tile's column sum has completed, a whole second pass later.  So the E_k copies,
            // the state rows and the gate product of tile i start on the first event and only the E_v copies wait for the
            // second one.
            if (i >= 2 && !__all_sync(0xffffffffu, mbar_wait(&bars->acc_empty[st], (uint32_t)((u - 1) & 1), abort_flag, 1))) break;
            // the slot ids are fetched first: a copy is a compiler barrier, so an id load between two copies would put a
            // shared-memory latency in front of every one of them
            int vj[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) vj[j] = ids_sh[i * TM + ((ptid + PROD_WARPS * 32 * j) >> 3)];
            if (i >= 1) issue_rows(Ek_st, a.Ek, i, vj);
            if (i >= 1) cp_commit();     // group E_k(i)
            {   // this thread's slot: state row (fetched an iteration ago) -> decayed fp16 row of the A tile (state / 64 folded into the exponent)
                const float dt = dts_sh[i * TM + prow];
                unsigned char* arow = A_sh + st * ATOM_BYTES + prow * 128;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {                    // chunks of 8 channels
                    const int ch = phalf * 4 + cc;
                    const float4 la = *reinterpret_cast<const float4*>(l2r_sh + ch * 8), lb = *reinterpret_cast<const float4*>(l2r_sh + ch * 8 + 4);
                    const float4 s0 = sr[2 * cc], s1 = sr[2 * cc + 1];
                    uint4 pk;
                    pk.x = pack_f16x2(s0.x * ex2_approx(fmaf(dt, la.x, -6.0f)), s0.y * ex2_approx(fmaf(dt, la.y, -6.0f)));
                    pk.y = pack_f16x2(s0.z * ex2_approx(fmaf(dt, la.z, -6.0f)), s0.w * ex2_approx(fmaf(dt, la.w, -6.0f)));
                    pk.z = pack_f16x2(s1.x * ex2_approx(fmaf(dt, lb.x, -6.0f)), s1.y * ex2_approx(fmaf(dt, lb.y, -6.0f)));
                    pk.w = pack_f16x2(s1.z * ex2_approx(fmaf(dt, lb.z, -6.0f)), s1.w * ex2_approx(fmaf(dt, lb.w, -6.0f)));
                    *reinterpret_cast<uint4*>(arow + ((ch ^ (prow & 7)) << 4)) = pk;
                }
                load_state(i + 1);                                  // in flight over the rest of this iteration and the next wait
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->a_full[st]);
            if (i >= 1) {                    // the E_v rows of tile i - 1 (every group but E_k(i)) have landed
                cp_wait<1>();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->ev_full[(i - 1) & 1]);
            }
            if (i >= 2 && !__all_sync(0xffffffffu, mbar_wait(&bars->pv_done[st], (uint32_t)((u - 1) & 1), abort_flag, 2))) break;
            if (i >= 1) issue_rows(Ev_st, a.Ev, i, vj);
            if (i >= 1) cp_commit();     // group E_v(i)
            done = i + 1;
            cp_wait<1>();                // E_k(i) has landed (E_v(i) may still be on its way)
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->acc_full[st]);
        }
        cp_wait<0>();
        __syncwarp();
        if (done > 0 && done == nt && lane == 0) mbar_arrive(&bars->ev_full[(nt - 1) & 1]);   // the last tile's E_v rows
    } else {
        // ============================================================ epilogue warps: a thread per slot and HALF a head (32 columns)
        // warp = half * 8 + head * 4 + TMEM lane quarter: four epilogue warps per scheduler instead of two.  The kernel is
        // latency-bound (short dependent chains between the tanh-bound gate pass, the maximum exchange and the operand
        // stores), so the extra warps are what fills the issue slots.
        const int head = (warp >> 2) & 1, half = warp >> 3;
        const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        uint32_t q2[HALF / 2];                                      // q / sqrt(hd) of this half head as packed bf16 pairs
#pragma unroll
        for (int j = 0; j < HALF / 2; ++j) q2[j] = pack_bf16x2(q_sh[head * HD + half * HALF + 2 * j], q_sh[head * HD + half * HALF + 2 * j + 1]);
        float m_run = -INFINITY, l_run = 0.f, o_run = 0.f;          // warps 0..3: running softmax state of output column `row`
        const int hc = row >> 6;                                    // ... which belongs to head hc of the pair
        const bool folder = warp < 4;
        auto fold = [&](int j) {        // tile j's column sums (its product has completed) into the running state
            const float* wr = wred + (j & 3) * 16;
            const float mt = wr[hc];
            const float lt = (wr[4 + hc * 4] + wr[4 + hc * 4 + 1]) + (wr[4 + hc * 4 + 2] + wr[4 + hc * 4 + 3]);
            const float v = tmem_ld_1(t_lane + (uint32_t)(COL_R + (j & 1) * 16));
            tmem_wait_ld();
            const float m_new = fmaxf(m_run, mt);
            const float c_old = __expf(m_run - m_new), c_new = __expf(mt - m_new);     // exp(-inf) = 0 on the first tile
            o_run = o_run * c_old + v * c_new;
            l_run = l_run * c_old + lt * c_new;
            m_run = m_new;
        };
        bool alive = true;
        for (int i = 0; i < nt; ++i) {
            const int st = i & 1, u = i >> 1;
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->acc_full[st], (uint32_t)(u & 1), abort_flag, 6))) { alive = false; break; }
            tc_fence_after_sync();
            const bool ok = ids_sh[i * TM + row] >= 0;
            const uint32_t t_acc = t_lane + (uint32_t)(st * ACC_COLS + head * HD + half * HALF);
            const unsigned char* ekrow = Ek_st + st * STAGE_BYTES + head * ATOM_BYTES + row * 128;
            unsigned char* evrow = Ev_st + st * STAGE_BYTES + head * ATOM_BYTES + row * 128;
            // ---- gate of this thread's 32 columns (kept) and its part of the score
            uint32_t g2[HALF / 2];                                  // packed bf16 pairs
            float sp0 = 0.f, sp1 = 0.f;
#pragma unroll
            for (int c = 0; c < HALF / 16; ++c) {                // 16 accumulator columns per load
                float pre[16];
                tmem_ld_32x32b_x16(t_acc + c * 16, pre);
                // the E_k chunks are loaded before the wait (a load after it could not be moved above it by the compiler)
                const uint4 eq[2] = {*reinterpret_cast<const uint4*>(ekrow + (((half * 4 + c * 2) ^ (row & 7)) << 4)),
                                     *reinterpret_cast<const uint4*>(ekrow + (((half * 4 + c * 2 + 1) ^ (row & 7)) << 4))};
                tmem_wait_ld();
#pragma unroll
                for (int j8 = 0; j8 < 2; ++j8) {
                    const uint32_t ew[4] = {eq[j8].x, eq[j8].y, eq[j8].z, eq[j8].w};
#pragma unroll
                    for (int pr = 0; pr < 4; ++pr) {
                        const int w = (c * 2 + j8) * 4 + pr;         // pair of columns within the half head
                        const float h0 = pre[j8 * 8 + pr * 2], h1 = pre[j8 * 8 + pr * 2 + 1];
                        const float g0 = SILU ? fmaf(h0, tanh_approx(h0), h0) : h0;
                        const float g1 = SILU ? fmaf(h1, tanh_approx(h1), h1) : h1;
                        g2[w] = pack_bf16x2(g0, g1);
                        // bf16 x bf16 products are exact in fp32, where the score is summed
                        fma_f32_bf16x2(sp0, sp1, g2[w], mul_bf16x2(q2[w], ew[pr]));
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->acc_empty[st]);       // accumulators read
            // ---- the rows' scores: both halves post their partial sums, the head's eight warps meet on an mbarrier (bounded)
            float* xb = xch + ((i & 1) * HPC + head) * 2 * TM;
            xb[half * TM + row] = ok ? sp0 + sp1 : -INFINITY;
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->hbar[head]);
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->hbar[head], (uint32_t)(i & 1), abort_flag, 8))) { alive = false; break; }
            const float s = xb[row] + xb[TM + row];
            // tile maximum of the head: every warp forms it from the 128 posted pairs (no second barrier)
            float mt = fmaxf(fmaxf(xb[lane] + xb[TM + lane], xb[32 + lane] + xb[TM + 32 + lane]),
                             fmaxf(xb[64 + lane] + xb[TM + 64 + lane], xb[96 + lane] + xb[TM + 96 + lane]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
            const float prob = ok ? __expf(s - mt) : 0.f;            // every tile holds at least one slot, so mt is finite
            const uint32_t p2 = pack_bf16x2(prob, prob);
            if (half == 0) {                                         // sums of p and the maximum, for the fold
                float* wr = wred + (i & 3) * 16;
                const float ps = warp_sum(prob);
                if (lane == 0) {
                    wr[4 + head * 4 + (warp & 3)] = ps;
                    if ((warp & 3) == 0) wr[head] = mt;
                }
            }
            // ---- (p * gate * E_v)[k, d] in bf16, over the E_v rows themselves, once they have landed (the four chunks' loads
            //      first: a store is a compiler barrier for the loads behind it)
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->ev_full[st], (uint32_t)(u & 1), abort_flag, 10))) { alive = false; break; }
            {
                uint4 ev4[4];
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) ev4[c4] = *reinterpret_cast<const uint4*>(evrow + (((half * 4 + c4) ^ (row & 7)) << 4));
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    const uint32_t ew[4] = {ev4[c4].x, ev4[c4].y, ev4[c4].z, ev4[c4].w};
                    uint32_t w[4];
#pragma unroll
                    for (int pr = 0; pr < 4; ++pr) w[pr] = ok ? mul_bf16x2(mul_bf16x2(g2[c4 * 4 + pr], p2), ew[pr]) : 0u;   // rows without a slot hold stale bytes
                    st_shared_v4(evrow + (((half * 4 + c4) ^ (row & 7)) << 4), w[0], w[1], w[2], w[3]);
                }
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->v_full[st]);          // operand rows (and this warp's sum, the head's maximum) are in place
            if (folder && i > 0) {      // fold tile i - 1 while the column sum of tile i is on its way
                if (!__all_sync(0xffffffffu, mbar_wait(&bars->pv_done[(i - 1) & 1], (uint32_t)(((i - 1) >> 1) & 1), abort_flag, 7))) { alive = false; break; }
                tc_fence_after_sync();
                fold(i - 1);
            }
        }
        if (folder && alive && nt > 0 &&
            __all_sync(0xffffffffu, mbar_wait(&bars->pv_done[(nt - 1) & 1], (uint32_t)(((nt - 1) >> 1) & 1), abort_flag, 7))) {
            tc_fence_after_sync();
            fold(nt - 1);
            float* part = a.part + (((size_t)b * (a.H / HPC) + hp) * a.S + split) * PART_FLOATS;
            part[row] = o_run;
            if ((row & 63) == 0) {
                part[ACC_COLS + hc] = m_run;
                part[ACC_COLS + 2 + hc] = l_run;
            }
        }
    }
    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == EPI_WARPS) {
        mbar_wait<100>(&bars->drain, 0u, &bars->drain_flag, 9);    // bounded: no product of this CTA is in flight when TMEM is released
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
    if (tid == 0 && (bars->abort_flag | bars->drain_flag)) atomicOr(status, bars->abort_flag | bars->drain_flag);   // sticky: never cleared by the library
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
