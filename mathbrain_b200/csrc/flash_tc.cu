// Flash-EMA gated cross-attention on the Blackwell tensor cores (MBEMA_MODE_TC_BF16), forward.
//
// One CTA owns (sample b, a 128-step time tile, a pair of heads) and loops over the sample's valid slots.
// Warp-specialised, 12 warps:
//   * four producer warps, each working on its own slots and its own pipeline stage (slot i belongs to producer warp
//     i % 4 and to stage i % 4), with no barrier between them.  For its slot the warp rebuilds the 128 x N state tile
//     A[t, :] = M_t[k, :] in shared memory (fp16 of state / 64, 128-byte-swizzled K-major rows; 11 significant bits
//     keep the pre-activations of slots with states in the hundreds accurate) as the packed product of the tile-start
//     snapshot and a table of decay powers, converts the slot's E_k / E_v rows to fp16, and one of its lanes issues
//         pre[128 x 128] = A[128 x N] @ (W_pe[:, 2 heads])        tcgen05.mma, fp32 accumulators in TMEM.
//     A warp's per-slot work is a chain of latencies (copy wait, barrier poll, shared-memory loads, proxy fence, UMMA
//     issue); four independent chains keep four slots in flight.  Because a producer warp owns its stage, it never
//     runs more than one barrier phase ahead of the epilogue (a parity wait cannot tell phases two apart).
//   * eight epilogue warps (a warpgroup per head): a thread owns one time step (its TMEM lane) and the head's 64
//     accumulator columns, reads them with tcgen05.ld and fuses SiLU, K = E_k*gate, V = E_v*gate, the score, the
//     online softmax and the P.V update, all thread-local.  One tanh per gate element is what the SM's
//     special-function pipe allows (16 per clock per SM, packed or not); the gate is formed in fp32 and packed to
//     fp16 pairs, the products with E_k, E_v and q are packed fp16 operations, and both the score terms and the P.V
//     terms are summed in fp32 with the mixed-precision FMA (one scheduler cycle per warp instruction, where a packed
//     16-bit FMA takes two: summing the score in packed fp16 first saved nothing and cost the unpacking).  The P.V
//     update of slot i - 1 shares the pass over the columns with the gate of slot i, and the softmax bookkeeping of
//     slot i - 1 runs under the TMEM load of slot i.
// A tiles and TMEM accumulators are four deep (all 512 TMEM columns) for N = 64.  Registers are rebalanced with
// setmaxnreg: 8*32*216 (epilogue) + 4*32*72 (producers) equals the launch allocation 384*168 (asking for more would
// block forever).  Hand-offs go through mbarriers with bounded waits; nothing in here spins without a limit, and a
// wait that gives up ends the CTA's loops, drains the tensor pipe and frees TMEM before the CTA leaves.
#include "flash.cuh"
#include <cuda_fp16.h>
#include "sm100_ptx.cuh"

namespace mbema {
namespace tc {

using namespace ptx;

static constexpr int TM = MBEMA_TILE_T;        // rows (time steps) per CTA
static constexpr int HPC = 2;                  // heads per CTA
static constexpr int HD = 64;
static constexpr int EPI_WARPS = 4 * HPC;            // 4 TMEM lane quarters x 2 heads
static constexpr int EPI_THREADS = 32 * EPI_WARPS;
static constexpr int PROD_WARPS = 4;
static constexpr int THREADS = EPI_THREADS + 32 * PROD_WARPS;
static constexpr int ATOM_BYTES = TM * 128;        // one 128-row x 64-column 16-bit swizzle atom
static constexpr int NSTAGE = PROD_WARPS;          // A-tile / accumulator stages: one per producer warp
static constexpr int NE = NSTAGE + 1;              // E-row stages: a slot's E_v row is read one slot later than its accumulators
static constexpr int ACC_COLS = HPC * HD;          // fp32 accumulator columns per stage
static constexpr int TMEM_COLS = 512;              // NSTAGE * ACC_COLS
static constexpr int MAX_SLOTS = 8192;
static constexpr float LAZY_MAX = 2.0f;            // the softmax reference maximum follows a score only beyond this margin
static constexpr int PDW = 2;                      // a producer warp prefetches this many of its own slots ahead
static constexpr int RW = PDW + 1;                 // ring stages per producer warp
static constexpr int RING_STAGE_BYTES = 256 + 2 * ACC_COLS * 4;   // fp16 snapshot row (N <= 128) + raw E_k, E_v rows
__host__ __device__ constexpr int r_stride(int N) { return N * 2; }

struct Smem {
    // offsets (bytes) into the dynamic shared memory block, base aligned to 1024
    int a_off, b_off, r_off, ts_off, e_off, ring_off, tok_off, slot_off, key_off, bar_off, total;
};

__host__ __device__ inline Smem smem_layout(int N, int K) {
    const int NK = N / 64;
    Smem s;
    int o = 0;
    s.a_off = o; o += NSTAGE * NK * ATOM_BYTES;
    s.b_off = o; o += NK * ATOM_BYTES;
    s.r_off = o; o += TM * r_stride(N);               // decay powers rho_n^r, fp16 [128][N]
    s.ts_off = o; o += NK == 1 ? TM * N * 2 : 0;      // N = 64: restart values (tok_state + 1) / 64 of the tile's steps, fp16
    s.e_off = o; o += NE * 2 * ACC_COLS * 2;          // E_k / E_v rows, fp16
    s.ring_off = o; o += PROD_WARPS * RW * RING_STAGE_BYTES;
    s.tok_off = o; o += TM * 4;
    s.slot_off = o; o += ((K * 2 + 15) / 16) * 16;
    s.key_off = o; o += ((K * 4 + 15) / 16) * 16;
    s.bar_off = o; o += 128;
    s.total = o + 1024;   // slack for the 1024-byte alignment of the base
    return s;
}

// byte offset of element (row, col) inside one swizzled 128-row x 64-col 16-bit atom
__device__ __forceinline__ int sw128_off(int row, int col) {
    return row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1));
}

struct Bars {
    uint64_t acc_full[NSTAGE];        // UMMAs of the stage done + E rows staged   (2 arrivals: commit, issuer)
    uint64_t acc_empty[NSTAGE];       // every epilogue warp has read the stage's accumulators (EPI_WARPS arrivals)
    uint64_t drain;                   // every issuing lane's UMMAs have completed (PROD_WARPS arrivals, teardown)
    uint32_t tmem_base;
    int abort_flag;
    unsigned spin_limit;         // poll limit of the waits (shortened by the test hook)
    int n_slots;
    int drain_flag;                   // give-up flag of the teardown wait (kept apart from abort_flag: that wait must not be cut short)
};

__device__ __forceinline__ uint4 mul4_f16x2(uint4 a, uint4 b) {
    return make_uint4(mul_f16x2(a.x, b.x), mul_f16x2(a.y, b.y), mul_f16x2(a.z, b.z), mul_f16x2(a.w, b.w));
}

// SILU is a compile-time switch: a run-time test inside the unrolled epilogue would put a branch between every
// pair of gate elements and stop the scheduler from overlapping their MUFU and FMA latencies.
// ROWS: slot-embedding rows are looked up through FlashArgs::erow (tables shared between samples)
template <bool SILU, int NK, bool ROWS>
__global__ void __launch_bounds__(THREADS, 1) k_flash_fwd_tc(FlashArgs a, int* status) {
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment for the swizzled operand tiles; the offset is added to the __shared__ array itself so that the
    // compiler keeps addressing shared memory directly (a pointer rebuilt from an integer would turn every access generic)
    unsigned char* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int N = NK * 64, RS = r_stride(N);
    const Smem L = smem_layout(N, a.K);
    unsigned char* A_sh = sm + L.a_off;
    unsigned char* B_sh = sm + L.b_off;
    unsigned char* R_sh = sm + L.r_off;                                        // fp16 [128][N]
    unsigned char* TS_sh = sm + L.ts_off;                                      // fp16 [128][64] (N = 64)
    __half* E2_sh = reinterpret_cast<__half*>(sm + L.e_off);                   // [stage][E_k | E_v][128 columns of the head pair]
    unsigned char* ring_sh = sm + L.ring_off;
    int* tok_sh = reinterpret_cast<int*>(sm + L.tok_off);
    unsigned short* slot_sh = reinterpret_cast<unsigned short*>(sm + L.slot_off);
    int* key_sh = reinterpret_cast<int*>(sm + L.key_off);
    Bars* bars = reinterpret_cast<Bars*>(sm + L.bar_off);
    volatile int* abort_flag = &bars->abort_flag;

    const int tile = blockIdx.x, hp = blockIdx.y, b = a.order ? a.order[blockIdx.z] : (int)blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int D = a.H * HD;
    const int t0 = tile * TM;
    const int Lb = a.seq_lens ? min(max(a.seq_lens[b], 0), a.T) : a.T;
    const bool is_epi = warp < EPI_WARPS;
    const int row = (warp & 3) * 32 + lane;         // time step within the tile (== TMEM lane for epilogue warps)
    const int t = t0 + row;

    if (t0 >= Lb) {   // whole tile beyond the valid length: define the outputs and leave (uniform per CTA)
        if (is_epi && t < a.T) {
            const int h = hp * HPC + (warp >> 2);
            const size_t qo = (((size_t)b * a.H + h) * a.T + t) * HD;
#pragma unroll
            for (int i = 0; i < HD; i += 4) *reinterpret_cast<float4*>(a.O + qo + i) = make_float4(0.f, 0.f, 0.f, 0.f);
            a.LSE[((size_t)b * a.H + h) * a.T + t] = 0.f;
        }
        return;
    }

    // ---------------------------------------------------------------- prologue (all 12 warps)
    if (tid == 0) {
        for (int i = 0; i < NSTAGE; ++i) {
            mbar_init(&bars->acc_full[i], 2);
            mbar_init(&bars->acc_empty[i], EPI_WARPS);
        }
        mbar_init(&bars->drain, PROD_WARPS);
        bars->abort_flag = *reinterpret_cast<volatile int*>(status);
        bars->spin_limit = a.test_withhold ? 64u : MBEMA_SPIN_LIMIT;   // an earlier CTA already gave up: do nothing
        bars->drain_flag = 0;
        fence_barrier_init();
    }
    if (warp == EPI_WARPS) {
        tmem_alloc(&bars->tmem_base, TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == EPI_WARPS + 1) {   // ordered compaction of the valid slots (index and key)
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
        // B operand: rows = the pair's 128 output columns, K-major over n, fp16 of 64 * W (the state operand carries
        // 1/64); 0.5 * W when the gate is SiLU (the epilogue evaluates SiLU(x) = h + h * tanh(h) with h = x / 2)
        const float wscale = (SILU ? 0.5f : 1.0f) * STATE_F16_UNSCALE;
        for (int i = tid; i < N * ACC_COLS; i += THREADS) {
            const int n = i / ACC_COLS, dd = i % ACC_COLS;
            const float w = a.W[(size_t)n * D + hp * ACC_COLS + dd] * wscale;
            *reinterpret_cast<__half*>(B_sh + (n >> 6) * ATOM_BYTES + sw128_off(dd, n & 63)) = __float2half_rn(w);
        }
        for (int i = tid; i < TM * N; i += THREADS) {   // decay powers rho_n^r, r = 0..127
            const int r = i / N, n = i % N;
            // N = 128: the backward kernel has no room for this table and forms rho^r as rho^(16 (r / 16)) * rho^(r % 16);
            // the same product here keeps the two kernels' state tiles identical
            const float l2 = log2f(a.rhos[n]);
            const float pw = NK == 1 ? exp2f((float)r * l2) : exp2f(16.0f * (float)(r >> 4) * l2) * exp2f((float)(r & 15) * l2);
            *reinterpret_cast<__half*>(R_sh + r * RS + n * 2) = __float2half_rn(pw);
        }
        for (int i = tid; i < TM; i += THREADS) {
            const int tt = t0 + i;
            tok_sh[i] = (tt < Lb) ? (int)(a.x[(size_t)b * a.T + tt] & 0x7fffffffLL) : -1;
        }
        if (NK == 1) {   // restart values of the tile's 128 steps: read from shared memory by the rows after an occurrence
            for (int i = tid; i < TM * (N / 4); i += THREADS) {
                const int r = i / (N / 4), c4 = i % (N / 4);
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (t0 + r < a.T) v = __ldg(reinterpret_cast<const float4*>(a.tok_state + ((size_t)b * a.T + t0 + r) * N) + c4);
                const float sc = STATE_F16_SCALE;                           // "+1": the occurrence itself
                reinterpret_cast<uint32_t*>(TS_sh)[2 * i] = pack_f16x2((v.x + 1.0f) * sc, (v.y + 1.0f) * sc);
                reinterpret_cast<uint32_t*>(TS_sh)[2 * i + 1] = pack_f16x2((v.z + 1.0f) * sc, (v.w + 1.0f) * sc);
            }
        }
        for (int i = tid; i < NE * 2 * ACC_COLS / 2; i += THREADS) reinterpret_cast<uint32_t*>(E2_sh)[i] = 0u;
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
        // ============================================================ producer warps: slot i belongs to warp i % 4
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        const int pw = warp - EPI_WARPS;
        const uint32_t idesc = umma_idesc_16(TM, ACC_COLS, 0, 0, 0, 0);          // fp16 operands, fp32 accumulation
        const uint32_t a_base = smem_u32(A_sh) + pw * NK * ATOM_BYTES, b_base = smem_u32(B_sh);
        constexpr int CH = N / 8;                   // 16-byte chunks per tile row
        constexpr int RPP = 32 / CH;                // tile rows the warp writes per pass
        constexpr int RB = 8;                       // passes whose loads are issued together
        const int cc = lane % CH, r0 = lane / CH;   // this lane's chunk column and first row
        const int esize = (a.e_dt == MBEMA_F32) ? 4 : 2;
        const int s_chunks = N / 8, e_chunks = ACC_COLS * esize / 16;     // 16-byte chunks per row (fp16 snapshot; raw E)
        const __half* snap16 = reinterpret_cast<const __half*>(a.tile_state + (size_t)a.B * a.nT * a.K * N);
        unsigned char* ring_w = ring_sh + pw * RW * RING_STAGE_BYTES;
        unsigned char* At = A_sh + pw * NK * ATOM_BYTES + (cc >> 3) * ATOM_BYTES;     // this warp's stage, this lane's atom
        const int c8 = cc & 7;
        const unsigned char* Rc = R_sh + cc * 16;
        // Asynchronous prefetch of slot i's snapshot row and raw E_k / E_v rows into this warp's ring stage `rs`.
        // E row of the next slot to prefetch (tables shared between samples): loaded one iteration ahead
        size_t erow_next = (ROWS && pw < n_slots) ? (size_t)a.erow[(size_t)b * a.K + slot_sh[pw]] : 0;
        auto prefetch = [&](int i, int rs) {
            if (i < n_slots) {
                const int k = slot_sh[i];
                const size_t er = ROWS ? erow_next : (size_t)b * a.K + k;
                if (ROWS && i + PROD_WARPS < n_slots) erow_next = (size_t)a.erow[(size_t)b * a.K + slot_sh[i + PROD_WARPS]];
                unsigned char* dst = ring_w + rs * RING_STAGE_BYTES;
                const unsigned char* srcS = reinterpret_cast<const unsigned char*>(snap16 + (((size_t)b * a.nT + tile) * a.K + k) * N);
                const size_t eoff = (er * D + hp * ACC_COLS) * esize;
                const unsigned char* srcK = reinterpret_cast<const unsigned char*>(a.Ek) + eoff;
                const unsigned char* srcV = reinterpret_cast<const unsigned char*>(a.Ev) + eoff;
                for (int c = lane; c < s_chunks + 2 * e_chunks; c += 32) {
                    const unsigned char* src;
                    unsigned char* d;
                    if (c < s_chunks) { src = srcS + c * 16; d = dst + c * 16; }
                    else if (c < s_chunks + e_chunks) { src = srcK + (c - s_chunks) * 16; d = dst + 256 + (c - s_chunks) * 16; }
                    else { src = srcV + (c - s_chunks - e_chunks) * 16; d = dst + 256 + ACC_COLS * 4 + (c - s_chunks - e_chunks) * 16; }
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(d)), "l"(src) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        for (int j = 0; j < PDW; ++j) prefetch(pw + PROD_WARPS * j, j);
        for (int i = pw, it = 0; i < n_slots; i += PROD_WARPS, ++it) {
            prefetch(i + PROD_WARPS * PDW, (it + PDW) % RW);
            asm volatile("cp.async.wait_group %0;" ::"n"(PDW) : "memory");   // this lane's copies for slot i have landed
            __syncwarp();                                                       // ... and so have the other lanes'
            // this warp's stage (A tile, accumulators) is free once the epilogue has read slot i - NSTAGE; by then the
            // epilogue is also done with the E rows of slot i - NE, whose stage the rows of slot i take
            if (it >= 1 && !mbar_wait(&bars->acc_empty[pw], (uint32_t)((it - 1) & 1), abort_flag, 1, &bars->spin_limit)) break;
            const int keyf = key_sh[i];
            const unsigned char* rg = ring_w + (it % RW) * RING_STAGE_BYTES;
            // E_k / E_v rows of the slot for the head pair, as fp16 (saturated): lane l converts columns 4l .. 4l+3 of both
            {
                uint2* dst = reinterpret_cast<uint2*>(E2_sh + (i % NE) * 2 * ACC_COLS) + lane;
                float4 fk, fv;
                if (esize == 4) {
                    fk = reinterpret_cast<const float4*>(rg + 256)[lane];
                    fv = reinterpret_cast<const float4*>(rg + 256 + ACC_COLS * 4)[lane];
                } else {
                    const uint2 rk = reinterpret_cast<const uint2*>(rg + 256)[lane];
                    const uint2 rv = reinterpret_cast<const uint2*>(rg + 256 + ACC_COLS * 4)[lane];
                    fk = make_float4(bf16_lo(rk.x), bf16_hi(rk.x), bf16_lo(rk.y), bf16_hi(rk.y));
                    fv = make_float4(bf16_lo(rv.x), bf16_hi(rv.x), bf16_lo(rv.y), bf16_hi(rv.y));
                }
                dst[0] = make_uint2(pack_f16x2_sat(fk.x, fk.y), pack_f16x2_sat(fk.z, fk.w));
                dst[ACC_COLS / 4] = make_uint2(pack_f16x2_sat(fv.x, fv.y), pack_f16x2_sat(fv.z, fv.w));
            }
            // The state tile: lane (cc, r0) writes chunk cc of rows r0, r0 + RPP, ...  The loads of RB passes are issued
            // together: the compiler cannot move a shared-memory load above an earlier shared-memory store (it cannot tell
            // the buffers apart), so a load-multiply-store loop would run as one load latency per pass.
            const uint4 sv = *reinterpret_cast<const uint4*>(rg + cc * 16);
            if (keyf >= 0) {
                // no occurrence of the slot's token in the tile: snapshot times decay power, one packed product per pair
                for (int rb = r0; rb < TM; rb += RPP * RB) {
                    uint4 rv[RB];
#pragma unroll
                    for (int j = 0; j < RB; ++j) rv[j] = *reinterpret_cast<const uint4*>(Rc + (rb + j * RPP) * RS);
#pragma unroll
                    for (int j = 0; j < RB; ++j) {
                        const int r = rb + j * RPP;
                        *reinterpret_cast<uint4*>(At + r * 128 + ((c8 ^ (r & 7)) << 4)) = mul4_f16x2(sv, rv[j]);
                    }
                }
            } else {
                // rows after an occurrence at step s restart from (tok_state[s] + 1) * rho^(r - s)
                const int key = keyf & 0x7fffffff;
                unsigned occ[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) occ[j] = __ballot_sync(0xffffffffu, tok_sh[32 * j + lane] == key);
                int s_have = -1;
                uint4 tv = make_uint4(0u, 0u, 0u, 0u);
                for (int r = r0; r < TM; r += RPP) {
                    const int wi = r >> 5, bi = r & 31;
                    int s = -1;
#pragma unroll
                    for (int j = 3; j >= 0; --j) {
                        const unsigned mm = (j > wi) ? 0u : (j == wi ? (occ[j] & ((1u << bi) - 1u)) : occ[j]);
                        if (s < 0 && mm) s = j * 32 + 31 - __clz(mm);
                    }
                    uint4 base = sv;
                    int rr = r;
                    if (s >= 0) {
                        if (s != s_have) {
                            if (NK == 1) {
                                tv = *reinterpret_cast<const uint4*>(TS_sh + s * 128 + cc * 16);
                            } else {
                                const float* src = a.tok_state + ((size_t)b * a.T + t0 + s) * N + cc * 8;
                                const float4 b0 = __ldg(reinterpret_cast<const float4*>(src));
                                const float4 b1 = __ldg(reinterpret_cast<const float4*>(src + 4));
                                const float sc = STATE_F16_SCALE;
                                tv = make_uint4(pack_f16x2((b0.x + 1.0f) * sc, (b0.y + 1.0f) * sc), pack_f16x2((b0.z + 1.0f) * sc, (b0.w + 1.0f) * sc),
                                                pack_f16x2((b1.x + 1.0f) * sc, (b1.y + 1.0f) * sc), pack_f16x2((b1.z + 1.0f) * sc, (b1.w + 1.0f) * sc));
                            }
                            s_have = s;
                        }
                        base = tv;
                        rr = r - s;
                    }
                    const uint4 rv = *reinterpret_cast<const uint4*>(Rc + rr * RS);
                    *reinterpret_cast<uint4*>(At + r * 128 + ((c8 ^ (r & 7)) << 4)) = mul4_f16x2(base, rv);
                }
            }
            fence_proxy_async_smem();
            __syncwarp();          // the whole tile and both E rows are in shared memory
            if (lane == 0) {
                tc_fence_after_sync();
#pragma unroll
                for (int k16 = 0; k16 < 4 * NK; ++k16) {     // contraction over n, 16 per instruction, 64 per swizzle atom
                    const int off = (k16 >> 2) * ATOM_BYTES + (k16 & 3) * 32;
                    umma_bf16_ss(tmem_base + (uint32_t)(pw * ACC_COLS), umma_desc_k_sw128(a_base + off), umma_desc_k_sw128(b_base + off),
                                 idesc, k16 != 0 ? 1u : 0u);
                }
                umma_commit(&bars->acc_full[pw]);   // first arrival: the UMMAs above have completed
                if (!(a.test_withhold && i == 0)) mbar_arrive(&bars->acc_full[pw]);   // second arrival: releases the staged E rows
                                                                                        // (test hook: withheld once)
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (lane == 0) umma_commit(&bars->drain);   // arrives once every UMMA this lane issued has completed
    } else {
        // ============================================================ epilogue warpgroups: a thread per time step, a head per warpgroup
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int wg = warp >> 2;
        const int h = hp * HPC + wg;
        const size_t qoff = (((size_t)b * a.H + h) * a.T + t) * HD;
        const bool row_ok = t < Lb;
        // q / sqrt(hd) and the gate of the previous slot as packed fp16 pairs; the output row in fp32
        uint32_t q2[HD / 2], g_old[HD / 2];
        float o[HD];
#pragma unroll
        for (int i = 0; i < HD; i += 4) {
            float4 v = row_ok ? ld4_dyn_f32(a.Q, a.q_dt, qoff + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            q2[i / 2] = pack_f16x2_sat(v.x * 0.125f, v.y * 0.125f);
            q2[i / 2 + 1] = pack_f16x2_sat(v.z * 0.125f, v.w * 0.125f);
            g_old[i / 2] = g_old[i / 2 + 1] = 0u;
            o[i] = o[i + 1] = o[i + 2] = o[i + 3] = 0.f;
        }
        const float rest = a.v_total - (float)a.kcount[b];
        float m, l;
        if (!a.listed_only && rest > 0.f) { m = 0.f; l = rest; } else { m = -INFINITY; l = 0.f; }
        const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(wg * HD);
        // In iteration i a thread
        //   (1) starts the TMEM load of slot i's accumulators,
        //   (2) under that load, finishes slot i - 1: updates the lazy softmax reference with score(i-1), gets p(i-1),
        //   (3) walks its 64 columns once, doing per pair of columns
        //         O += p(i-1) * (E_v(i-1) * gate(i-1))                                    P.V, one slot behind
        //         gate(i) = SiLU(pre) = h + h * tanh(h), h = pre (W_pe carries the 1/2)    overwrites gate(i-1)
        //         score(i) += gate(i) * (q * E_k(i))                                       summed in fp32 (mixed-precision FMA)
        // The reference maximum only moves when a score exceeds it by more than LAZY_MAX (the probabilities stay below
        // e^LAZY_MAX, well inside fp16), so rescaling the output row is rare.
        float s_prev = 0.f;                     // score(i-1)
        bool alive = true;
        // (2): softmax bookkeeping of a finished slot with score s; returns its probability in both fp16 halves
        auto finish_slot = [&](float s) -> uint32_t {
            if (s > m + LAZY_MAX) {
                const float alpha = __expf(m - s);     // m = -inf at the start: alpha = 0
                l *= alpha;
#pragma unroll
                for (int j = 0; j < HD; ++j) o[j] *= alpha;
                m = s;
            }
            const float p = __expf(s - m);
            l += p;
            return pack_f16x2(p, p);
        };
        for (int i = 0; i < n_slots; ++i) {
            const int st = i % NSTAGE, u = i / NSTAGE;
            alive = mbar_wait(&bars->acc_full[st], (uint32_t)(u & 1), abort_flag, 2, &bars->spin_limit);
            if (!alive) break;
            tc_fence_after_sync();
            const uint32_t t_acc = t_lane + st * ACC_COLS;
            float pre[2][16];
            tmem_ld_32x32b_x16(t_acc, pre[0]);
            const uint32_t p2 = (i >= 1) ? finish_slot(s_prev) : 0u;
            // (3)
            const uint32_t* ek2 = reinterpret_cast<const uint32_t*>(E2_sh + (i % NE) * 2 * ACC_COLS + wg * HD);
            const uint32_t* ev2 = reinterpret_cast<const uint32_t*>(E2_sh + ((i + NE - 1) % NE) * 2 * ACC_COLS + ACC_COLS + wg * HD);
            float sp0 = 0.f, sp1 = 0.f;
#pragma unroll
            for (int c = 0; c < HD / 16; ++c) {      // 16 accumulator columns (8 pairs) per TMEM load, the next load in flight
                // the E-row broadcasts are issued before the wait (a load after it could not be moved above it by the compiler)
                const uint4 ekA = *reinterpret_cast<const uint4*>(ek2 + c * 8), ekB = *reinterpret_cast<const uint4*>(ek2 + c * 8 + 4);
                const uint4 evA = *reinterpret_cast<const uint4*>(ev2 + c * 8), evB = *reinterpret_cast<const uint4*>(ev2 + c * 8 + 4);
                tmem_wait_ld();
                if (c + 1 < HD / 16) tmem_ld_32x32b_x16(t_acc + (c + 1) * 16, pre[(c + 1) & 1]);
                const uint32_t ekw[8] = {ekA.x, ekA.y, ekA.z, ekA.w, ekB.x, ekB.y, ekB.z, ekB.w};
                const uint32_t evw[8] = {evA.x, evA.y, evA.z, evA.w, evB.x, evB.y, evB.z, evB.w};
                // software pipeline over the pairs: the two tanh of pair j + 1 are issued between the FMA-pipe work of pair j
                float tA, tB;
                asm volatile("tanh.approx.f32 %0, %1;" : "=f"(tA) : "f"(pre[c & 1][0]));
                asm volatile("tanh.approx.f32 %0, %1;" : "=f"(tB) : "f"(pre[c & 1][1]));
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int w = c * 8 + j;
                    const float h0 = pre[c & 1][2 * j], h1 = pre[c & 1][2 * j + 1];
                    const float t0v = tA, t1v = tB;
                    if (j + 1 < 8) asm volatile("tanh.approx.f32 %0, %1;" : "=f"(tA) : "f"(pre[c & 1][2 * j + 2]));
                    {
                        const uint32_t gv = mul_f16x2(g_old[w], evw[j]);
                        asm volatile("{\n\t.reg .b16 xl, xh, yl, yh;\n\tmov.b32 {xl, xh}, %2;\n\tmov.b32 {yl, yh}, %3;\n\t"
                                     "fma.rn.f32.f16 %0, xl, yl, %0;\n\tfma.rn.f32.f16 %1, xh, yh, %1;\n\t}"
                                     : "+f"(o[2 * w]), "+f"(o[2 * w + 1]) : "r"(gv), "r"(p2));
                    }
                    if (j + 1 < 8) asm volatile("tanh.approx.f32 %0, %1;" : "=f"(tB) : "f"(pre[c & 1][2 * j + 3]));
                    const float g0 = SILU ? fmaf(h0, t0v, h0) : h0;
                    const float g1 = SILU ? fmaf(h1, t1v, h1) : h1;
                    const uint32_t gg = pack_f16x2(g0, g1);
                    g_old[w] = gg;
                    const uint32_t qe = mul_f16x2(q2[w], ekw[j]);
                    asm volatile("{\n\t.reg .b16 xl, xh, yl, yh;\n\tmov.b32 {xl, xh}, %2;\n\tmov.b32 {yl, yh}, %3;\n\t"
                                 "fma.rn.f32.f16 %0, xl, yl, %0;\n\tfma.rn.f32.f16 %1, xh, yh, %1;\n\t}"
                                 : "+f"(sp0), "+f"(sp1) : "r"(gg), "r"(qe));
                }
            }
            // the stage's accumulators are consumed (its E rows live in their own, deeper ring)
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->acc_empty[st]);
            s_prev = sp0 + sp1;
        }
        if (alive && n_slots > 0) {
            // the last slot: its softmax bookkeeping and P.V update
            const uint32_t p2 = finish_slot(s_prev);
            const uint32_t* ev2 = reinterpret_cast<const uint32_t*>(E2_sh + ((n_slots - 1) % NE) * 2 * ACC_COLS + ACC_COLS + wg * HD);
#pragma unroll
            for (int w4 = 0; w4 < HD / 2; w4 += 4) {
                const uint4 evp = *reinterpret_cast<const uint4*>(ev2 + w4);
                const uint32_t evw[4] = {evp.x, evp.y, evp.z, evp.w};
#pragma unroll
                for (int pr = 0; pr < 4; ++pr) fma_f32_f16x2(o[2 * (w4 + pr)], o[2 * (w4 + pr) + 1], mul_f16x2(g_old[w4 + pr], evw[pr]), p2);
            }
        }
        if (alive && t < a.T) {
            const float inv = (row_ok && l > 0.f) ? 1.0f / l : 0.f;
#pragma unroll
            for (int i = 0; i < HD; i += 4)
                *reinterpret_cast<float4*>(a.O + qoff + i) = make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
            a.LSE[((size_t)b * a.H + h) * a.T + t] = (row_ok && l > 0.f) ? m + logf(l) : 0.f;
        }
    }
    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == EPI_WARPS) {
        mbar_wait<100>(&bars->drain, 0u, &bars->drain_flag, 3);   // bounded: no UMMA of this CTA is in flight when TMEM is released
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (tid == 0 && (bars->abort_flag | bars->drain_flag)) atomicOr(status, bars->abort_flag | bars->drain_flag);   // sticky: later CTAs of this launch skip their work
}

}  // namespace tc

bool flash_tc_supported(int H, int N, int K) {
    return (H % tc::HPC) == 0 && (N == 64 || N == 128) && K <= tc::MAX_SLOTS && tc::smem_layout(N, K).total <= 227 * 1024;
}

size_t flash_fwd_tc_ws() { return 256; }

int flash_fwd_tc(const FlashArgs& a, void* ws, cudaStream_t st) {
    int* status = reinterpret_cast<int*>((reinterpret_cast<uintptr_t>(ws) + 15) & ~uintptr_t(15));
    const tc::Smem L = tc::smem_layout(a.N, a.K);
    dim3 grid(a.nT, a.H / tc::HPC, a.B);
#define MBEMA_LAUNCH_FWD(S_, NK_, R_)                                                                                     \
    do {                                                                                                             \
        MBEMA_CUDA_TRY(cudaFuncSetAttribute(tc::k_flash_fwd_tc<S_, NK_, R_>, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total)); \
        tc::k_flash_fwd_tc<S_, NK_, R_><<<grid, tc::THREADS, L.total, st>>>(a, status);                                 \
    } while (0)
    const bool rows = a.erow != nullptr;
#define MBEMA_PICK(R_)                                                                     \
    do {                                                                                   \
        if (a.N == 64) { if (a.silu) MBEMA_LAUNCH_FWD(true, 1, R_); else MBEMA_LAUNCH_FWD(false, 1, R_); }             \
        else { if (a.silu) MBEMA_LAUNCH_FWD(true, 2, R_); else MBEMA_LAUNCH_FWD(false, 2, R_); }                       \
    } while (0)
    if (rows) MBEMA_PICK(true); else MBEMA_PICK(false);
#undef MBEMA_PICK
#undef MBEMA_LAUNCH_FWD
    return check_launch();
}

}  // namespace mbema
