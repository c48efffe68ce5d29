// Flash-EMA gated cross-attention on the Blackwell tensor cores (MBEMA_MODE_TC_BF16), backward.
//
// Same decomposition as the forward (CTA = sample x 128-step tile x head pair, loop over the valid slots, producer
// warpgroup + two epilogue warpgroups, a thread per time step), with three tensor-core products per slot:
//   (1) pre[128 t x 128 d]  = A[t, n] @ W[n, d]                      recompute of the gate pre-activation
//   (2) dW^T[128 d x N]    += dpre[t, d]^T @ A[t, n]                 accumulated in TMEM over all slots of the CTA
//   (3) dE_k[d], dE_v[d]    = (ds*q*g)[t, d]^T @ 1,  (p*dO*g)[t, d]^T @ 1     column sums over the tile's time steps
// For N = 64 product (1) takes fp16 operands (state / 64, W * 64; see flash_tc.cu) and product (2) bf16 ones, so the
// producer stores every state tile twice (fp16, and the same values converted to bf16).
// The epilogue threads read the accumulators of (1) once, in 16-column chunks: pass 1 forms the gate and its
// derivative (fp32, kept as packed bf16 pairs), the score and dO.V, giving p = exp(s - LSE) and ds; pass 2 builds the
// three bf16 operand tiles of (2) and (3) in packed bf16 arithmetic and writes them to shared memory
// (128-byte-swizzled, "MN-major": the tile row is the time step, which is the contraction index).  dQ is
// accumulated in the thread's own TMEM lane (tcgen05.ld / tcgen05.st), which keeps 64 registers free; q and dO are
// held as packed bf16 pairs.  Every wait is bounded (see sm100_ptx.cuh).
#include "flash.cuh"
#include <cuda_fp16.h>
#include "sm100_ptx.cuh"

namespace mbema {
namespace tcb {

using namespace ptx;

static constexpr int TM = MBEMA_TILE_T;
static constexpr int HPC = 2;
static constexpr int HD = 64;
static constexpr int EPI_WARPS = 4 * HPC;
static constexpr int EPI_THREADS = 32 * EPI_WARPS;
static constexpr int PROD_THREADS = 128;
static constexpr int THREADS = EPI_THREADS + PROD_THREADS;
static constexpr int ATOM_BYTES = TM * 128;
static constexpr int ACC_COLS = HPC * HD;
// Per channel count N = 64 * NK (NK = 1, 2): stages and the TMEM map
//   NK = 1: gate 2 x 128 | dW^T 64  | dE_k 16 | dE_v 16 | ... | dQ 128 at column 384
//   NK = 2: gate 1 x 128 | dW^T 128 | dE_k 16 | dE_v 16 | ... | decay powers 64 at column 320 | dQ 128 at column 384
template <int NK> struct Cfg {
    static constexpr int N = 64 * NK;
    static constexpr int NA = 2;                       // A-tile / E-row stages in shared memory (32 KB each, see STAGE_BYTES)
    static constexpr int NACC = NK == 1 ? 2 : 1;       // gate accumulator stages in TMEM
    static constexpr int COL_DW = NACC * ACC_COLS;     // dW^T [128 d x N]
    static constexpr int COL_DEK = COL_DW + N;         // dE_k column sums (16 columns, all equal)
    static constexpr int COL_DEV = COL_DEK + 16;
    static constexpr int COL_DQ = 384;                 // dQ accumulators [128 t x (2 heads x 64)] fp32, one row per thread
    static constexpr int COL_RT = 320;                 // NK = 2 only: the row's decay powers as 64 packed fp16 pairs (columns 320..383 are free there)
};
static constexpr int TMEM_COLS = 512;
// every producer warp prefetches into its own ring: the slot's fp16 snapshot row (N <= 128) and the 32 columns of E_k / E_v
// that its lanes convert (fp32 at most); PD slots ahead (N = 128 has shared memory for two stages only)
__host__ __device__ constexpr int prefetch_dist(int NK) { return NK == 1 ? 3 : 1; }
static constexpr int RING_STAGE_BYTES = 256 + 2 * 32 * 4;
static constexpr int MAX_SLOTS = 4096;

struct Smem {
    int a_off, b_off, z_off, ones_off, r_off, e2_off, ring_off, tok_off, slot_off, key_off, bar_off, total;
};

__host__ __device__ inline Smem smem_layout(int K, int NK) {
    const int NA = 2;
    Smem s;
    int o = 0;
    s.a_off = o; o += NA * 2 * ATOM_BYTES;        // N = 64: fp16 tile (gate product) + bf16 tile (dW product); N = 128: two bf16 atoms
    s.b_off = o; o += NK * ATOM_BYTES;            // W^T for the gate product (K-major over n)
    s.z_off = o; o += 3 * HPC * ATOM_BYTES;       // dpre, ds*q*g, p*dO*g tiles: [kind][head][128 t][64 d] bf16
    s.ones_off = o; o += 2048;                    // 16 x 64 bf16 ones (B operand of the column sums)
    // decay powers rho_n^r.  NK = 1: bf16 table [128][64] (the forward kernel multiplies bf16 snapshots by bf16 powers;
    // the recompute must build bit-identical state tiles or p = exp(s - LSE) stops summing to one);
    // NK = 2: fp32, two levels [8][128] (r / 16) and [16][128] (r % 16), product rounded once like the forward's fp32 table
    s.r_off = o; o += NK == 1 ? TM * 64 * 2 : 24 * 128 * 4;
    s.e2_off = o; o += NA * 2 * ACC_COLS * 2;     // E_k / E_v rows as bf16 (operands of the packed epilogue arithmetic)
    s.ring_off = o; o += 4 * (prefetch_dist(NK) + 1) * RING_STAGE_BYTES;
    s.tok_off = o; o += TM * 4;
    s.slot_off = o; o += ((K * 2 + 15) / 16) * 16;
    s.key_off = o; o += ((K * 4 + 15) / 16) * 16;
    s.bar_off = o; o += 256;
    s.total = o + 1024;
    return s;
}

__device__ __forceinline__ int sw128_off(int row, int col) {
    return row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1));
}

struct Bars {
    uint64_t acc_full[2];        // gate UMMAs done + E rows staged                  (2 arrivals)
    uint64_t acc_empty[2];       // all epilogue warps finished reading the stage      (EPI_WARPS arrivals)
    uint64_t z_full;             // all epilogue warps wrote their part of the Z tiles (EPI_WARPS arrivals)
    uint64_t z_done;             // products (2) and (3) of the slot have completed    (3 arrivals: one commit per issuing warp)
    uint64_t drain;              // every issuing lane's UMMAs have completed (4 arrivals, teardown)
    uint32_t tmem_base;
    int abort_flag;
    unsigned spin_limit;         // poll limit of the waits (shortened by the test hook)
    int drain_flag;              // give-up flag of the teardown wait (apart from abort_flag: that wait must not be cut short)
    int n_slots;
    unsigned dmax_bits;          // largest |dO| among the CTA's rows (bit pattern of a non-negative float)
};

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ float tmem_ld_1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    return __uint_as_float(r);
}

// ROWS: slot-embedding rows are looked up through FlashArgs::erow (tables shared between samples)
template <bool SILU, int NK, bool ROWS>
__global__ void __launch_bounds__(THREADS, 1) k_flash_bwd_tc(FlashArgs a, int* status) {
    constexpr int N = Cfg<NK>::N, NA = Cfg<NK>::NA, NACC = Cfg<NK>::NACC;
    constexpr int COL_DW = Cfg<NK>::COL_DW, COL_DEK = Cfg<NK>::COL_DEK, COL_DEV = Cfg<NK>::COL_DEV, COL_DQ = Cfg<NK>::COL_DQ, COL_RT = Cfg<NK>::COL_RT;
    constexpr int STAGE_BYTES = 2 * ATOM_BYTES;
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment for the swizzled operand tiles; the offset is added to the __shared__ array itself so that the
    // compiler keeps addressing shared memory directly (a pointer rebuilt from an integer would turn every access generic)
    unsigned char* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const Smem L = smem_layout(a.K, NK);
    unsigned char* A_sh = sm + L.a_off;
    unsigned char* B_sh = sm + L.b_off;
    unsigned char* Z_sh = sm + L.z_off;
    unsigned char* ones_sh = sm + L.ones_off;
    float* R_sh = reinterpret_cast<float*>(sm + L.r_off);                       // NK = 2
    __nv_bfloat16* Rb_sh = reinterpret_cast<__nv_bfloat16*>(sm + L.r_off);      // NK = 1
    __nv_bfloat16* E2_sh = reinterpret_cast<__nv_bfloat16*>(sm + L.e2_off);
    unsigned char* ring_sh = sm + L.ring_off;
    int* tok_sh = reinterpret_cast<int*>(sm + L.tok_off);
    unsigned short* slot_sh = reinterpret_cast<unsigned short*>(sm + L.slot_off);
    int* key_sh = reinterpret_cast<int*>(sm + L.key_off);
    Bars* bars = reinterpret_cast<Bars*>(sm + L.bar_off);
    uint64_t* a_free = reinterpret_cast<uint64_t*>(sm + L.bar_off + 96);   // [NA] A/E stage released by product (2)
    uint64_t* a_full = reinterpret_cast<uint64_t*>(sm + L.bar_off + 128);  // [NA] every producer warp has written its rows of the tile and its E columns (4 arrivals)
    volatile int* abort_flag = &bars->abort_flag;

    const int tile = blockIdx.x, hp = blockIdx.y, b = a.order ? a.order[blockIdx.z] : (int)blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int D = a.H * HD;
    const int t0 = tile * TM;
    const int Lb = a.seq_lens ? min(max(a.seq_lens[b], 0), a.T) : a.T;
    const bool is_epi = warp < EPI_WARPS;
    const int row = (warp & 3) * 32 + lane;
    const int t = t0 + row;
    float* part_out = a.dW_part + (((size_t)b * (a.H / HPC) + hp) * a.nT + tile) * (size_t)N * ACC_COLS;   // [n][128 d]

    if (t0 >= Lb) {   // nothing to do for this tile: zero dQ rows and the dW partial (uniform per CTA)
        if (is_epi && t < a.T) {
            const int h = hp * HPC + (warp >> 2);
            const size_t qo = (((size_t)b * a.H + h) * a.T + t) * HD;
#pragma unroll
            for (int i = 0; i < HD; i += 4) *reinterpret_cast<float4*>(a.dQ + qo + i) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int i = tid; i < N * ACC_COLS; i += THREADS) part_out[i] = 0.f;
        return;
    }

    // ---------------------------------------------------------------- prologue
    if (tid == 0) {
        for (int i = 0; i < NACC; ++i) {
            mbar_init(&bars->acc_full[i], 2);
            mbar_init(&bars->acc_empty[i], EPI_WARPS);
        }
        for (int i = 0; i < NA; ++i) {
            mbar_init(&a_free[i], 1);
            mbar_init(&a_full[i], 4);
        }
        mbar_init(&bars->z_full, EPI_WARPS);
        mbar_init(&bars->z_done, 3);
        mbar_init(&bars->drain, 4);
        bars->drain_flag = 0;
        bars->abort_flag = *reinterpret_cast<volatile int*>(status);
        bars->spin_limit = a.test_withhold ? 64u : MBEMA_SPIN_LIMIT;
        bars->dmax_bits = 0u;
        fence_barrier_init();
    }
    if (warp == EPI_WARPS) {
        tmem_alloc(&bars->tmem_base, TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == EPI_WARPS + 1) {
        int n = 0;
        for (int k0 = 0; k0 < a.K; k0 += 32) {
            const int k = k0 + lane;
            const long long kv = (k < a.K) ? a.unique[(size_t)b * a.K + k] : -1;
            const bool ok = kv >= 0;
            const unsigned m = __ballot_sync(0xffffffffu, ok);
            if (ok) {
                const int pos = n + __popc(m & ((1u << lane) - 1u));
                slot_sh[pos] = (unsigned short)k;
                key_sh[pos] = (int)(kv & 0x7fffffffLL);
            }
            n += __popc(m);
        }
        if (lane == 0) bars->n_slots = n;
    }
    {
        const float wscale = SILU ? 0.5f : 1.0f;
        for (int i = tid; i < N * ACC_COLS; i += THREADS) {
            const int n = i / ACC_COLS, dd = i % ACC_COLS;
            const float w = a.W[(size_t)n * D + hp * ACC_COLS + dd] * wscale;
            unsigned char* dstw = B_sh + (n >> 6) * ATOM_BYTES + sw128_off(dd, n & 63);
            *reinterpret_cast<__half*>(dstw) = __float2half_rn(w * STATE_F16_UNSCALE);   // the state operand carries 1/64
        }
        if (NK == 1) {
            for (int i = tid; i < TM * N; i += THREADS) {
                const int r = i / N, n = i % N;
                reinterpret_cast<__half*>(Rb_sh)[i] = __float2half_rn(exp2f((float)r * log2f(a.rhos[n])));   // fp16 powers, as the forward
            }
        } else {   // rho^r = rho^(16 (r / 16)) * rho^(r % 16): rows 0..7 hold the first factor, rows 8..23 the second
            for (int i = tid; i < 24 * N; i += THREADS) {
                const int r = i / N, n = i % N;
                const float e = (r < 8) ? 16.0f * (float)r : (float)(r - 8);
                R_sh[i] = exp2f(e * log2f(a.rhos[n]));
            }
        }
        for (int i = tid; i < 1024; i += THREADS) reinterpret_cast<__nv_bfloat16*>(ones_sh)[i] = __float2bfloat16(1.0f);
        for (int i = tid; i < TM; i += THREADS) {
            const int tt = t0 + i;
            tok_sh[i] = (tt < Lb) ? (int)(a.x[(size_t)b * a.T + tt] & 0x7fffffffLL) : -1;
        }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;
    const int n_slots = bars->abort_flag ? 0 : bars->n_slots;
    // bit 31 of a slot's key: its token occurs among the tile's 128 steps (only those slots have restart rows)
    for (int pos = tid; pos < n_slots; pos += THREADS) {
        const int key = key_sh[pos];
        bool hot = false;
#pragma unroll 8
        for (int j = 0; j < TM; j += 4) {
            const int4 tk = *reinterpret_cast<const int4*>(tok_sh + j);
            hot |= (tk.x == key) | (tk.y == key) | (tk.z == key) | (tk.w == key);
        }
        if (hot) key_sh[pos] = key | (int)0x80000000u;
    }
    __syncthreads();

    if (!is_epi) {
        // ============================================================ producer warpgroup
        asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
        // The gate product takes an fp16 state tile (state / 64) and fp16 W (W * 64): 11 significant bits, where bf16
        // operands moved the pre-activations of slots with states in the hundreds by ~0.1.  The dW product reads the same
        // tile: its rounding errors are the same for many consecutive time steps of a slot (the state decays slowly), so
        // they do not average out over the sum, and 8 significant bits cost 2 % in dW_pe on small batches.  dpre, the
        // other operand, is therefore fp16 as well, scaled by a power of two chosen per CTA from its rows of dO.
        const uint32_t idesc_gate = umma_idesc_16(TM, ACC_COLS, 0, 0, 0, 0);            // A, B K-major, fp16
        const uint32_t idesc_dw = umma_idesc_16(ACC_COLS, N, 1, 1, 0, 0);               // A = dpre (MN-major), B = state tile (MN-major), both fp16
        const uint32_t idesc_de = umma_idesc_bf16(ACC_COLS, 16, 1, 0);        // A = Z tile (MN-major), B = ones (K-major)
        const uint32_t a_base = smem_u32(A_sh), b_base = smem_u32(B_sh), z_base = smem_u32(Z_sh), o_base = smem_u32(ones_sh);
        const int wi = row >> 5, bi = row & 31;
        const int pwarp = warp - EPI_WARPS;
        constexpr int PD = prefetch_dist(NK), RING = PD + 1;
        const int esize = (a.e_dt == MBEMA_F32) ? 4 : 2;
        const int s_chunks = N / 8, e_chunks = 32 * esize / 16;      // 16-byte chunks: snapshot row; this warp's 32 columns of E_k (E_v)
        const __half* snap16 = reinterpret_cast<const __half*>(a.tile_state + (size_t)a.B * a.nT * a.K * N);
        unsigned char* ring_w = ring_sh + pwarp * RING * RING_STAGE_BYTES;
        // The producer warps do not wait for one another: each prefetches what its own lanes need (the whole snapshot row,
        // read as broadcasts, and 32 columns of the E rows) and reports its part of the tile on an mbarrier.
        // E row of the next slot to prefetch (tables shared between samples: one index load per slot, a slot ahead)
        size_t erow_next = (ROWS && n_slots > 0) ? (size_t)a.erow[(size_t)b * a.K + slot_sh[0]] : 0;
        auto prefetch = [&](int j) {
            if (j < n_slots) {
                const int k = slot_sh[j];
                const size_t er = ROWS ? erow_next : (size_t)b * a.K + k;
                if (ROWS && j + 1 < n_slots) erow_next = (size_t)a.erow[(size_t)b * a.K + slot_sh[j + 1]];
                if (lane < s_chunks + 2 * e_chunks) {
                    unsigned char* dst = ring_w + (j % RING) * RING_STAGE_BYTES;
                    const size_t eoff = (er * D + hp * ACC_COLS + pwarp * 32) * esize;
                    const unsigned char* src;
                    unsigned char* d;
                    if (lane < s_chunks) {
                        src = reinterpret_cast<const unsigned char*>(snap16 + (((size_t)b * a.nT + tile) * a.K + k) * N) + lane * 16;
                        d = dst + lane * 16;
                    } else if (lane < s_chunks + e_chunks) {
                        src = reinterpret_cast<const unsigned char*>(a.Ek) + eoff + (lane - s_chunks) * 16;
                        d = dst + 256 + (lane - s_chunks) * 16;
                    } else {
                        src = reinterpret_cast<const unsigned char*>(a.Ev) + eoff + (lane - s_chunks - e_chunks) * 16;
                        d = dst + 256 + 128 + (lane - s_chunks - e_chunks) * 16;
                    }
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(d)), "l"(src) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        // products (2) and (3) of slot j, once the epilogue has written the Z tiles.  Issuing a UMMA costs its thread
        // on the order of a hundred cycles, so the 24 instructions are spread over three warps (dW^T, dE_k, dE_v;
        // the gate product has the fourth), each committing its own group.
        const uint64_t d_zp = umma_desc_mn_sw128(z_base + 0 * HPC * ATOM_BYTES, ATOM_BYTES, 1024);
        const uint64_t d_zk = umma_desc_mn_sw128(z_base + 1 * HPC * ATOM_BYTES, ATOM_BYTES, 1024);
        const uint64_t d_zv = umma_desc_mn_sw128(z_base + 2 * HPC * ATOM_BYTES, ATOM_BYTES, 1024);
        const uint64_t d_ones = umma_desc_k_sw128(o_base);
        const uint64_t d_a0 = umma_desc_mn_sw128(a_base, ATOM_BYTES, 1024);
        const uint64_t d_ak0 = umma_desc_k_sw128(a_base), d_b0 = umma_desc_k_sw128(b_base);
        const int role = warp - EPI_WARPS;          // 0: gate, 1: dW^T, 2: dE_k, 3: dE_v
        auto issue_grad_products = [&](int j) {
            mbar_wait(&bars->z_full, (uint32_t)(j & 1), abort_flag, 1, &bars->spin_limit);
            tc_fence_after_sync();
            if (role == 1) {
                const uint64_t d_at = d_a0 + (uint64_t)(((j % NA) * STAGE_BYTES) >> 4);
#pragma unroll
                for (int ks = 0; ks < TM / 16; ++ks)      // contraction over the 128 time steps, 16 per instruction
                    umma_bf16_ss(tmem_base + COL_DW, d_zp + (uint64_t)(ks * (2048 >> 4)), d_at + (uint64_t)(ks * (2048 >> 4)),
                                 idesc_dw, (j | ks) != 0 ? 1u : 0u);
                umma_commit(&bars->z_done);
                umma_commit(&a_free[j % NA]);
            } else {
                const uint64_t dz = (role == 2) ? d_zk : d_zv;
                const uint32_t col = (role == 2) ? COL_DEK : COL_DEV;
#pragma unroll
                for (int ks = 0; ks < TM / 16; ++ks)
                    umma_bf16_ss(tmem_base + col, dz + (uint64_t)(ks * (2048 >> 4)), d_ones, idesc_de, ks != 0 ? 1u : 0u);
                umma_commit(&bars->z_done);
            }
        };
        // NK = 2: decay powers rho^r for 8 consecutive channels starting at n0 (r = steps since the reference state) from the
        // two-level fp32 table; the forward kernel fills its fp16 table with the same products, so both build the same tiles
        auto decay8 = [&](int r, int n0, float* out) {
            const float* hi = R_sh + (r >> 4) * N + n0;
            const float* lo = R_sh + (8 + (r & 15)) * N + n0;
            const float4 h0 = *reinterpret_cast<const float4*>(hi), h1 = *reinterpret_cast<const float4*>(hi + 4);
            const float4 l0 = *reinterpret_cast<const float4*>(lo), l1 = *reinterpret_cast<const float4*>(lo + 4);
            out[0] = h0.x * l0.x; out[1] = h0.y * l0.y; out[2] = h0.z * l0.z; out[3] = h0.w * l0.w;
            out[4] = h1.x * l1.x; out[5] = h1.y * l1.y; out[6] = h1.z * l1.z; out[7] = h1.w * l1.w;
        };
        // NK = 1: this row's powers as packed fp16 pairs, register-resident (cold rows: packed multiply, as the forward)
        uint32_t R2[NK == 1 ? 32 : 1];
        if (NK == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) R2[j] = *reinterpret_cast<const uint32_t*>(Rb_sh + row * N + 2 * j);
        }
        // NK = 2: this row's 128 powers as packed fp16 pairs do not fit the registers, and rebuilding them from the two-level
        // table for every slot (four 16-byte table loads, eight multiplies and four conversions per eight channels) made the
        // producers the critical path.  They are built once and parked in 64 unused TMEM columns of the thread's own lane;
        // a slot reads them back with four tcgen05.ld.  Same values as before: fp16 of the fp32 two-level product.
        const uint32_t t_rt = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)COL_RT;
        if (NK == 2) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float buf[16];
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    float rr[8];
                    decay8(row, (q * 4 + c4) * 8, rr);
                    buf[c4 * 4 + 0] = __uint_as_float(pack_f16x2(rr[0], rr[1]));
                    buf[c4 * 4 + 1] = __uint_as_float(pack_f16x2(rr[2], rr[3]));
                    buf[c4 * 4 + 2] = __uint_as_float(pack_f16x2(rr[4], rr[5]));
                    buf[c4 * 4 + 3] = __uint_as_float(pack_f16x2(rr[6], rr[7]));
                }
                tmem_st_32x32b_x16(t_rt + q * 16, buf);
            }
            tmem_wait_st();
        }
        for (int j = 0; j < PD; ++j) prefetch(j);
        for (int i = 0; i < n_slots; ++i) {
            const int sa = i % NA, sc = i % NACC;
            prefetch(i + PD);
            asm volatile("cp.async.wait_group %0;" ::"n"(PD) : "memory");   // this lane's copies for slot i have landed
            __syncwarp();                                                      // ... and so have the other lanes'
            if (i >= NA && !__all_sync(0xffffffffu, mbar_wait(&a_free[sa], (uint32_t)((i / NA - 1) & 1), abort_flag, 2, &bars->spin_limit))) break;   // gave up (the whole warp leaves together): drain and leave
            const int keyf = key_sh[i];
            const int key = keyf & 0x7fffffff;
            const unsigned char* rg = ring_w + (i % RING) * RING_STAGE_BYTES;
            {   // column `row` of the head pair's E_k / E_v rows, as bf16
                float ekv, evv;
                if (esize == 4) {
                    ekv = reinterpret_cast<const float*>(rg + 256)[lane];
                    evv = reinterpret_cast<const float*>(rg + 256 + 128)[lane];
                } else {
                    ekv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(rg + 256)[lane]);
                    evv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(rg + 256 + 128)[lane]);
                }
                E2_sh[sa * 2 * ACC_COLS + row] = __float2bfloat16(ekv);
                E2_sh[sa * 2 * ACC_COLS + ACC_COLS + row] = __float2bfloat16(evv);
            }
            int s = -1;
            if (keyf < 0) {
                unsigned w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) w[j] = __ballot_sync(0xffffffffu, tok_sh[32 * j + lane] == key);
#pragma unroll
                for (int j = 3; j >= 0; --j) {
                    unsigned mm = (j > wi) ? 0u : (j == wi ? (w[j] & ((1u << bi) - 1u)) : w[j]);
                    if (s < 0 && mm) s = j * 32 + 31 - __clz(mm);
                }
            }
            unsigned char* Arow = A_sh + sa * STAGE_BYTES + row * 128;
            if (NK == 2) {
                // every lane builds the cold row (snapshot times parked powers; the TMEM loads are warp-wide), lanes whose
                // token occurs in the tile overwrite it below
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float rv[16];
                    tmem_ld_32x32b_x16(t_rt + q * 16, rv);
                    uint4 sv[4];
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4) sv[c4] = *reinterpret_cast<const uint4*>(rg + (q * 4 + c4) * 16);
                    tmem_wait_ld();
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4) {
                        const int cc = q * 4 + c4;
                        uint4 pk;
                        pk.x = mul_f16x2(sv[c4].x, __float_as_uint(rv[c4 * 4 + 0]));
                        pk.y = mul_f16x2(sv[c4].y, __float_as_uint(rv[c4 * 4 + 1]));
                        pk.z = mul_f16x2(sv[c4].z, __float_as_uint(rv[c4 * 4 + 2]));
                        pk.w = mul_f16x2(sv[c4].w, __float_as_uint(rv[c4 * 4 + 3]));
                        *reinterpret_cast<uint4*>(Arow + (cc >> 3) * ATOM_BYTES + (((cc & 7) ^ (row & 7)) << 4)) = pk;
                    }
                }
            }
            if (s >= 0) {   // restart from the token's own state at its last in-tile occurrence (+1)
                const float* base = a.tok_state + ((size_t)b * a.T + t0 + s) * N;
#pragma unroll 2
                for (int cc = 0; cc < N / 8; ++cc) {
                    const float4 b0 = __ldg(reinterpret_cast<const float4*>(base + cc * 8));
                    const float4 b1 = __ldg(reinterpret_cast<const float4*>(base + cc * 8 + 4));
                    const float sc = STATE_F16_SCALE;
                    uint4 pk;     // as the forward: fp16 restart value x fp16 power, packed multiply
                    pk.x = pack_f16x2((b0.x + 1.0f) * sc, (b0.y + 1.0f) * sc);
                    pk.y = pack_f16x2((b0.z + 1.0f) * sc, (b0.w + 1.0f) * sc);
                    pk.z = pack_f16x2((b1.x + 1.0f) * sc, (b1.y + 1.0f) * sc);
                    pk.w = pack_f16x2((b1.z + 1.0f) * sc, (b1.w + 1.0f) * sc);
                    uint4 rv;
                    if (NK == 1) {
                        rv = *reinterpret_cast<const uint4*>(Rb_sh + (row - s) * N + cc * 8);
                    } else {
                        float rr[8];
                        decay8(row - s, cc * 8, rr);
                        rv = make_uint4(pack_f16x2(rr[0], rr[1]), pack_f16x2(rr[2], rr[3]), pack_f16x2(rr[4], rr[5]), pack_f16x2(rr[6], rr[7]));
                    }
                    pk.x = mul_f16x2(pk.x, rv.x); pk.y = mul_f16x2(pk.y, rv.y); pk.z = mul_f16x2(pk.z, rv.z); pk.w = mul_f16x2(pk.w, rv.w);
                    *reinterpret_cast<uint4*>(Arow + (cc >> 3) * ATOM_BYTES + (((cc & 7) ^ (row & 7)) << 4)) = pk;
                }
            } else if (NK == 1) {
                // snapshot times decay power.  All loads come first: the compiler cannot move a shared-memory load above an
                // earlier shared-memory store (it cannot tell the buffers apart), so a load-multiply-store loop would run as
                // N / 8 load latencies in a row.
                uint4 svv[N / 8];
#pragma unroll
                for (int cc = 0; cc < N / 8; ++cc) svv[cc] = *reinterpret_cast<const uint4*>(rg + cc * 16);
                if (NK == 2) {
#pragma unroll
                    for (int cc = 0; cc < N / 8; ++cc) {
                        float rr[8];
                        decay8(row, cc * 8, rr);
                        svv[cc].x = mul_f16x2(svv[cc].x, pack_f16x2(rr[0], rr[1]));
                        svv[cc].y = mul_f16x2(svv[cc].y, pack_f16x2(rr[2], rr[3]));
                        svv[cc].z = mul_f16x2(svv[cc].z, pack_f16x2(rr[4], rr[5]));
                        svv[cc].w = mul_f16x2(svv[cc].w, pack_f16x2(rr[6], rr[7]));
                    }
                } else {
#pragma unroll
                    for (int cc = 0; cc < N / 8; ++cc) {
                        svv[cc].x = mul_f16x2(svv[cc].x, R2[(4 * cc) & 31]);
                        svv[cc].y = mul_f16x2(svv[cc].y, R2[(4 * cc + 1) & 31]);
                        svv[cc].z = mul_f16x2(svv[cc].z, R2[(4 * cc + 2) & 31]);
                        svv[cc].w = mul_f16x2(svv[cc].w, R2[(4 * cc + 3) & 31]);
                    }
                }
#pragma unroll
                for (int cc = 0; cc < N / 8; ++cc) {
                    const uint4 pk = svv[cc];
                    *reinterpret_cast<uint4*>(Arow + (cc >> 3) * ATOM_BYTES + (((cc & 7) ^ (row & 7)) << 4)) = pk;
                }
            }
            fence_proxy_async_smem();
            __syncwarp();          // this warp's 32 rows of the tile and its E columns are in shared memory
            if (lane == 0) mbar_arrive(&a_full[sa]);
            if (lane == 0) {
                if (role == 0) {
                    mbar_wait(&a_full[sa], (uint32_t)((i / NA) & 1), abort_flag, 3, &bars->spin_limit);    // all four warps' rows and E columns
                    if (i >= NACC) mbar_wait(&bars->acc_empty[sc], (uint32_t)((i / NACC - 1) & 1), abort_flag, 4, &bars->spin_limit);
                    tc_fence_after_sync();
#pragma unroll
                    for (int k16 = 0; k16 < 4 * NK; ++k16) {     // contraction over n, 16 per instruction, 64 per swizzle atom
                        const int off = (k16 >> 2) * ATOM_BYTES + (k16 & 3) * 32;
                        umma_bf16_ss(tmem_base + (uint32_t)(sc * ACC_COLS), d_ak0 + (uint64_t)((sa * STAGE_BYTES + off) >> 4),
                                     d_b0 + (uint64_t)(off >> 4), idesc_gate, k16 != 0 ? 1u : 0u);
                    }
                    umma_commit(&bars->acc_full[sc]);
                    if (!(a.test_withhold && i == 0)) mbar_arrive(&bars->acc_full[sc]);   // withheld once by the test hook
                } else if (i >= 1) {
                    issue_grad_products(i - 1);
                }
            }
            __syncwarp();
        }
        if (lane == 0 && role != 0 && n_slots > 0 && !*abort_flag) issue_grad_products(n_slots - 1);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (lane == 0) umma_commit(&bars->drain);    // arrives once every UMMA this lane issued has completed
    } else {
        // ============================================================ epilogue warpgroups: a thread per time step, a head per warpgroup
        asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
        const int wg = warp >> 2;
        const int h = hp * HPC + wg;
        const size_t qoff = (((size_t)b * a.H + h) * a.T + t) * HD;
        const bool row_ok = t < Lb;
        uint32_t q2[HD / 2], do2[HD / 2];     // q / sqrt(hd) and dO as packed bf16 pairs
        float drow = 0.f, dmx = 0.f;
#pragma unroll
        for (int i = 0; i < HD; i += 4) {
            const float4 v = row_ok ? ld4_dyn_f32(a.Q, a.q_dt, qoff + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 g = row_ok ? ld4_dyn_f32(a.dO, a.do_dt, qoff + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 ov = row_ok ? *reinterpret_cast<const float4*>(a.O + qoff + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            q2[i / 2] = pack_bf16x2(v.x * 0.125f, v.y * 0.125f);
            q2[i / 2 + 1] = pack_bf16x2(v.z * 0.125f, v.w * 0.125f);
            do2[i / 2] = pack_bf16x2(g.x, g.y);
            do2[i / 2 + 1] = pack_bf16x2(g.z, g.w);
            drow += g.x * ov.x + g.y * ov.y + g.z * ov.z + g.w * ov.w;
            dmx = fmaxf(dmx, fmaxf(fmaxf(fabsf(g.x), fabsf(g.y)), fmaxf(fabsf(g.z), fabsf(g.w))));
        }
        const float lse = row_ok ? a.LSE[((size_t)b * a.H + h) * a.T + t] : 0.f;
        // dpre enters the dW product as fp16, scaled by a power of two chosen per CTA.  dpre is of the size of p * dO times
        // factors of order one (gate derivative, E rows, q), and p = exp(score - LSE) is of the size of exp(-LSE) for
        // scores of a few units, so the scale puts the CTA's largest |dO| * exp(-LSE) at 4: terms 2^-16 below the typical
        // size keep their full precision, and there are 14 binades of room above it before fp16 saturates.
        dmx = row_ok ? dmx * __expf(fminf(fmaxf(-lse, -80.0f), 80.0f)) : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dmx = fmaxf(dmx, __shfl_xor_sync(0xffffffffu, dmx, o));
        if (lane == 0) atomicMax(&bars->dmax_bits, __float_as_uint(dmx));
        named_bar_sync(3, EPI_THREADS);
        float sigma = 1.0f;
        {
            const float mx = __uint_as_float(*reinterpret_cast<volatile unsigned*>(&bars->dmax_bits));
            int e = 0;
            if (mx > 1.0e-36f && mx < 1.0e36f) { frexpf(mx, &e); sigma = ldexpf(1.0f, 2 - e); }
        }
        const float hs = 0.5f * sigma;
        const uint32_t hs2 = pack_bf16x2(hs, hs), nhs2 = pack_bf16x2(-hs, -hs), sig2 = pack_bf16x2(sigma, sigma);   // powers of two: exact
        const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t t_dq = t_lane + (uint32_t)(COL_DQ + wg * HD);
        {
            float z16[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) z16[j] = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_st_32x32b_x16(t_dq + c * 16, z16);
            tmem_wait_st();
        }
        const uint32_t zr = smem_u32(Z_sh + wg * ATOM_BYTES + row * 128) | (uint32_t)((row & 7) << 4);   // shared-window address of the Z row, swizzle term folded in; + kind * HPC * ATOM_BYTES
        float* dE_out = (wg == 0 ? a.dEk : a.dEv) + hp * ACC_COLS + row;   // + E row of the slot * D
        size_t de_row_prev = 0;                                          // E row of slot i - 1
        const uint32_t t_de = t_lane + (wg == 0 ? COL_DEK : COL_DEV);

        bool alive = true;
        for (int i = 0; i < n_slots; ++i) {
            const int sa = i % NA, sc = i % NACC;
            size_t de_row_cur = 0;                                      // used one iteration later: the load has a whole slot to land
            if (ROWS) de_row_cur = (size_t)a.erow[(size_t)b * a.K + slot_sh[i]];
            if (!mbar_wait(&bars->acc_full[sc], (uint32_t)((i / NACC) & 1), abort_flag, 5, &bars->spin_limit)) { alive = false; break; }
            tc_fence_after_sync();
            const uint32_t t_acc = t_lane + (uint32_t)(sc * ACC_COLS + wg * HD);
            // ---- pass 1: gate, its derivative, score and dO.V; gate and derivative are kept as packed bf16 pairs
            uint32_t g2[HD / 2], dsl2[HD / 2];
            float sp[2] = {0.f, 0.f}, dpp[2] = {0.f, 0.f};
            const uint32_t* ek2a = reinterpret_cast<const uint32_t*>(E2_sh + sa * 2 * ACC_COLS + wg * HD);
            const uint32_t* ev2a = ek2a + ACC_COLS / 2;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float pre[16];
                tmem_ld_32x32b_x16(t_acc + c * 16, pre);
                // the E-row broadcasts are issued before the wait (a load after it could not be moved above it by the compiler)
                const uint4 ekq[2] = {*reinterpret_cast<const uint4*>(ek2a + c * 8), *reinterpret_cast<const uint4*>(ek2a + c * 8 + 4)};
                const uint4 evq[2] = {*reinterpret_cast<const uint4*>(ev2a + c * 8), *reinterpret_cast<const uint4*>(ev2a + c * 8 + 4)};
                tmem_wait_ld();
#pragma unroll
                for (int j8 = 0; j8 < 2; ++j8) {
                    const int w0 = c * 8 + j8 * 4;
                    const uint4 ekp = ekq[j8];
                    const uint4 evp = evq[j8];
                    const uint32_t ekw[4] = {ekp.x, ekp.y, ekp.z, ekp.w}, evw[4] = {evp.x, evp.y, evp.z, evp.w};
#pragma unroll
                    for (int pr = 0; pr < 4; ++pr) {
                        uint32_t gg, dd;
                        {   // gate and derivative in fp32 (packing the pre-activation first costs 2-3x in dW_pe accuracy), then packed
                            float g[2], th[2];
#pragma unroll
                            for (int v = 0; v < 2; ++v) {
                                const float hh = pre[j8 * 8 + pr * 2 + v];
                                th[v] = SILU ? tanh_approx(hh) : 0.f;
                                g[v] = SILU ? fmaf(hh, th[v], hh) : hh;       // h = x / 2, th = tanh(h): SiLU = h + h*th
                            }
                            gg = pack_bf16x2(g[0], g[1]);
                            if (SILU) {     // sg = sigmoid(x) = (1 + th)/2, SiLU' = sg + SiLU*(1 - sg); times sigma, in packed bf16 from the fp32 tanh
                                const uint32_t th2 = pack_bf16x2(th[0], th[1]);
                                dd = fma_bf16x2(gg, fma_bf16x2(nhs2, th2, hs2), fma_bf16x2(hs2, th2, hs2));
                            } else {
                                dd = sig2;
                            }
                        }
                        g2[w0 + pr] = gg;
                        dsl2[w0 + pr] = dd;
                        // score and dO.V terms: bf16 x bf16 products are exact in fp32, where they are summed
                        fma_f32_bf16x2(sp[0], sp[1], gg, mul_bf16x2(q2[w0 + pr], ekw[pr]));
                        fma_f32_bf16x2(dpp[0], dpp[1], gg, mul_bf16x2(do2[w0 + pr], evw[pr]));
                    }
                }
            }
            // the gate accumulators have been read: the next gate product may overwrite the stage while pass 2 runs
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->acc_empty[sc]);
            const float s = sp[0] + sp[1];
            const float p = row_ok ? __expf(s - lse) : 0.f;
            const float dsr = p * ((dpp[0] + dpp[1]) - drow);     // d loss / d score
            const float dsq = dsr * 0.125f;
            const uint32_t dsr2 = pack_bf16x2(dsr, dsr), p2 = pack_bf16x2(p, p), dsq2 = pack_bf16x2(dsq, dsq);
            // ---- column sums of the previous slot (also: its Z tiles have been consumed)
            if (i >= 1) {
                if (!mbar_wait(&bars->z_done, (uint32_t)((i - 1) & 1), abort_flag, 6, &bars->spin_limit)) { alive = false; break; }
                tc_fence_after_sync();
                const float v = tmem_ld_1(t_de);
                tmem_wait_ld();
                atomicAdd(dE_out + (ROWS ? de_row_prev : (size_t)b * a.K + slot_sh[i - 1]) * D, v);
            }
            // ---- pass 2: operand tiles of the dW / dE products in packed bf16 arithmetic, dQ in fp32 (TMEM)
            const uint32_t* ek2 = reinterpret_cast<const uint32_t*>(E2_sh + sa * 2 * ACC_COLS + wg * HD);
            const uint32_t* ev2 = ek2 + ACC_COLS / 2;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float dq[16];
                tmem_ld_32x32b_x16(t_dq + c * 16, dq);
#pragma unroll
                for (int j8 = 0; j8 < 2; ++j8) {          // 8 columns -> one 16-byte chunk per tile
                    const int w0 = (c * 16 + j8 * 8) / 2;   // first packed pair of the chunk
                    const uint4 ekp = *reinterpret_cast<const uint4*>(ek2 + w0);
                    const uint4 evp = *reinterpret_cast<const uint4*>(ev2 + w0);
                    const uint32_t ekw[4] = {ekp.x, ekp.y, ekp.z, ekp.w}, evw[4] = {evp.x, evp.y, evp.z, evp.w};
                    uint32_t zp[4], zk[4], zv[4], ge[4];
#pragma unroll
                    for (int pr = 0; pr < 4; ++pr) {
                        const uint32_t gg = g2[w0 + pr];
                        const uint32_t aq = mul_bf16x2(dsr2, q2[w0 + pr]);                // ds * q
                        const uint32_t bd = mul_bf16x2(p2, do2[w0 + pr]);                 // p * dO
                        zk[pr] = mul_bf16x2(aq, gg);                                      // ds * q * g
                        zv[pr] = mul_bf16x2(bd, gg);                                      // p * dO * g
                        {   // sigma * dgate * SiLU' -> fp16: the last product exactly in fp32 (mixed-precision FMA), one conversion
                            float z0 = 0.f, z1 = 0.f;
                            fma_f32_bf16x2(z0, z1, fma_bf16x2(bd, evw[pr], mul_bf16x2(aq, ekw[pr])), dsl2[w0 + pr]);
                            zp[pr] = pack_f16x2_sat(z0, z1);
                        }
                        ge[pr] = mul_bf16x2(gg, ekw[pr]);                                 // K = g * E_k, for dQ
                    }
                    // swizzled chunk address: the row base has bits 4..6 clear, so base + ((k ^ r) << 4) == (base | r << 4) ^ (k << 4)
                    const uint32_t za = zr ^ (uint32_t)((c * 2 + j8) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(za), "r"(zp[0]), "r"(zp[1]), "r"(zp[2]), "r"(zp[3]) : "memory");
                    asm volatile("st.shared.v4.b32 [%0+%5], {%1, %2, %3, %4};" ::"r"(za), "r"(zk[0]), "r"(zk[1]), "r"(zk[2]), "r"(zk[3]), "n"(1 * HPC * ATOM_BYTES) : "memory");
                    asm volatile("st.shared.v4.b32 [%0+%5], {%1, %2, %3, %4};" ::"r"(za), "r"(zv[0]), "r"(zv[1]), "r"(zv[2]), "r"(zv[3]), "n"(2 * HPC * ATOM_BYTES) : "memory");
                    if (j8 == 0) tmem_wait_ld();
#pragma unroll
                    for (int pr = 0; pr < 4; ++pr)      // dq += (ds / 8) * K in fp32: bf16 x bf16 products are exact
                        fma_f32_bf16x2(dq[j8 * 8 + pr * 2], dq[j8 * 8 + pr * 2 + 1], ge[pr], dsq2);
                }
                tmem_st_32x32b_x16(t_dq + c * 16, dq);
            }
            tmem_wait_st();
            fence_proxy_async_smem();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->z_full);
            if (ROWS) de_row_prev = de_row_cur;
        }
        if (n_slots > 0 && alive && mbar_wait(&bars->z_done, (uint32_t)((n_slots - 1) & 1), abort_flag, 7, &bars->spin_limit)) {
            tc_fence_after_sync();
            const float v = tmem_ld_1(t_de);
            tmem_wait_ld();
            atomicAdd(dE_out + (ROWS ? de_row_prev : (size_t)b * a.K + slot_sh[n_slots - 1]) * D, v);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float dq[16];
            tmem_ld_32x32b_x16(t_dq + c * 16, dq);
            tmem_wait_ld();
            if (t < a.T && !*abort_flag) {      // after a give-up nothing of this CTA is stored (the status word says so)
#pragma unroll
                for (int i = 0; i < 16; i += 4)
                    *reinterpret_cast<float4*>(a.dQ + qoff + c * 16 + i) = make_float4(dq[i], dq[i + 1], dq[i + 2], dq[i + 3]);
            }
        }
        if (wg == 0) {   // dW^T accumulator: lane = column d of the head pair, TMEM columns = n
            float acc[32];
#pragma unroll
            for (int c = 0; c < N / 32; ++c) {
                if (n_slots > 0 && !*abort_flag) {
                    tmem_ld_32x32b_x32(t_lane + COL_DW + c * 32, acc);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[j] = 0.f;
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) part_out[(size_t)(c * 32 + j) * ACC_COLS + row] = acc[j] * (STATE_F16_UNSCALE / sigma);
            }
        }
    }
    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == EPI_WARPS) {
        mbar_wait<100>(&bars->drain, 0u, &bars->drain_flag, 8);    // bounded: no UMMA of this CTA is in flight when TMEM is released
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (tid == 0 && (bars->abort_flag | bars->drain_flag)) atomicOr(status, bars->abort_flag | bars->drain_flag);   // sticky: never cleared by the library
}

// dW[n, hp*128 + d] = sum over (b, tile) of part[b][hp][tile][n][d]      (fixed order -> deterministic)
__global__ void k_flash_dw_reduce_tc(const float* __restrict__ part, float* __restrict__ dW, int B, int HP, int nT, int D, int N) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N * D) return;
    const int n = idx / D, col = idx % D, hp = col / ACC_COLS, d = col % ACC_COLS;
    float s = 0.f;
    for (int b = 0; b < B; ++b)
        for (int tl = 0; tl < nT; ++tl)
            s += part[((((size_t)b * HP + hp) * nT + tl) * N + n) * ACC_COLS + d];
    dW[(size_t)n * D + col] = s;
}

}  // namespace tcb

bool flash_bwd_tc_supported(int H, int N, int K) {
    return (H % tcb::HPC) == 0 && (N == 64 || N == 128) && K <= tcb::MAX_SLOTS && tcb::smem_layout(K, N / 64).total <= 227 * 1024;
}

size_t flash_bwd_tc_ws(int64_t B, int64_t H, int64_t T, int64_t N) {
    const int64_t nT = (T + MBEMA_TILE_T - 1) / MBEMA_TILE_T;
    return 256 + (size_t)(B * (H / tcb::HPC) * nT) * N * tcb::ACC_COLS * sizeof(float) + 256;
}

int flash_bwd_tc(FlashArgs a, float* dW, void* ws, cudaStream_t st) {
    const int D = a.H * tcb::HD;
    int* status = reinterpret_cast<int*>((reinterpret_cast<uintptr_t>(ws) + 255) & ~uintptr_t(255));
    a.dW_part = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(status) + 256);
    MBEMA_CUDA_TRY(cudaMemsetAsync(a.dEk, 0, (size_t)a.e_rows * D * sizeof(float), st));
    MBEMA_CUDA_TRY(cudaMemsetAsync(a.dEv, 0, (size_t)a.e_rows * D * sizeof(float), st));
    const tcb::Smem L = tcb::smem_layout(a.K, a.N / 64);
    dim3 grid(a.nT, a.H / tcb::HPC, a.B);
#define MBEMA_LAUNCH_BWD(S_, NK_, R_)                                                                                     \
    do {                                                                                                             \
        MBEMA_CUDA_TRY(cudaFuncSetAttribute(tcb::k_flash_bwd_tc<S_, NK_, R_>, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total)); \
        tcb::k_flash_bwd_tc<S_, NK_, R_><<<grid, tcb::THREADS, L.total, st>>>(a, status);                               \
    } while (0)
    const bool rows = a.erow != nullptr;
#define MBEMA_PICK(R_)                                                                     \
    do {                                                                                   \
        if (a.N == 64) { if (a.silu) MBEMA_LAUNCH_BWD(true, 1, R_); else MBEMA_LAUNCH_BWD(false, 1, R_); }             \
        else { if (a.silu) MBEMA_LAUNCH_BWD(true, 2, R_); else MBEMA_LAUNCH_BWD(false, 2, R_); }                       \
    } while (0)
    if (rows) MBEMA_PICK(true); else MBEMA_PICK(false);
#undef MBEMA_PICK
#undef MBEMA_LAUNCH_BWD
    int rc = check_launch();
    if (rc) return rc;
    const int total = a.N * D;
    tcb::k_flash_dw_reduce_tc<<<(total + 255) / 256, 256, 0, st>>>(a.dW_part, dW, a.B, a.H / tcb::HPC, a.nT, D, a.N);
    return check_launch();
}

}  // namespace mbema
