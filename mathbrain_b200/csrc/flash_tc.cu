// Flash-EMA gated cross-attention on the Blackwell tensor cores (MBEMA_MODE_TC_BF16), forward.
//
// One CTA owns (sample b, a 128-step time tile, a pair of heads) and loops over the sample's valid slots.
// Warp-specialised, 12 warps:
//   * producer warpgroup (warps 8-11, one thread per time step): for slot k rebuilds the 128 x N state tile
//     A[t, :] = M_t[k, :] (16-bit, 128-byte-swizzled K-major rows: fp16 of state / 64 for N = 64, whose 11
//     significant bits keep the pre-activations of slots with states in the hundreds accurate, bf16 for N = 128)
//     in shared memory from the tile-start snapshot and
//     a table of decay powers, stages the slot's E_k / E_v rows as fp32, and one of its threads issues
//         pre[128 x 128] = A[128 x N] @ (W_pe[:, 2 heads])        tcgen05.mma, fp32 accumulators in TMEM;
//   * two epilogue warpgroups (a warpgroup per head, a thread per time step) read their 64 accumulator columns
//     with tcgen05.ld and fuse SiLU, K = E_k*gate, V = E_v*gate, the score, the online softmax and the P.V update,
//     all thread-local.
// A tiles and TMEM accumulators are multi-buffered, so state generation and the tensor core run ahead of the
// epilogue.  Registers are rebalanced with setmaxnreg (epilogue threads hold q, the output row and 64 accumulator
// columns; the per-CTA total, 8*32*216 + 4*32*72, equals the launch allocation 384*168).  Hand-offs go through
// mbarriers with bounded waits; nothing in here spins without a limit.
#include "flash.cuh"
#include <cuda_fp16.h>
#include "sm100_ptx.cuh"

namespace mbema {
namespace tc {

using namespace ptx;

static constexpr int TM = MBEMA_TILE_T;        // rows (time steps) per CTA
static constexpr int HPC = 2;                  // heads per CTA
static constexpr int HD = 64;
static constexpr int EPI_WARPS = 4 * HPC;
static constexpr int EPI_THREADS = 32 * EPI_WARPS;
static constexpr int PROD_THREADS = 128;
static constexpr int THREADS = EPI_THREADS + PROD_THREADS;
static constexpr int ATOM_BYTES = TM * 128;        // one 128-row x 64-column bf16 swizzle atom
static constexpr int NSTAGE_MAX = 4;               // A-tile / accumulator / E-row pipeline depth: 4 stages for N = 64 (all
                                                   // 512 TMEM columns), 3 for N = 128 (shared memory)
__host__ __device__ constexpr int nstage(int NK) { return NK == 1 ? 4 : 3; }
static constexpr int ACC_COLS = HPC * HD;          // fp32 accumulator columns per stage
static constexpr int TMEM_COLS = 512;              // power of two >= stages * ACC_COLS
static constexpr int MAX_SLOTS = 8192;
static constexpr int PD = 3;                       // prefetch distance (slots) of the snapshot / E-row ring
static constexpr int RING = PD + 1;
static constexpr int RING_STAGE_BYTES = 128 * 4 + 2 * ACC_COLS * 4;   // snapshot row (N <= 128 fp32) + raw E_k, E_v rows

struct Smem {
    // offsets (bytes) into the dynamic shared memory block, base aligned to 1024
    int a_off, b_off, r_off, e_off, ring_off, ts_off, tok_off, slot_off, key_off, bar_off, total;
};

__host__ __device__ inline Smem smem_layout(int N, int K) {
    const int NK = N / 64;
    Smem s;
    int o = 0;
    const int NSTAGE = nstage(NK);
    s.a_off = o; o += NSTAGE * NK * ATOM_BYTES;
    s.b_off = o; o += NK * ATOM_BYTES;
    s.r_off = o; o += NK == 1 ? TM * 64 * 2 : TM * (N + 4) * 4;   // decay powers rho_n^r: bf16 [128][64] (N = 64) or fp32
    s.e_off = o; o += NSTAGE * 2 * HPC * HD * 4;
    s.ring_off = o; o += RING * RING_STAGE_BYTES;
    s.ts_off = o; o += NK == 1 ? TM * 64 * 2 : 0;  // N = 64: restart values (tok_state + 1) of the tile's 128 steps, bf16
    s.tok_off = o; o += TM * 4;
    s.slot_off = o; o += ((K * 2 + 15) / 16) * 16;
    s.key_off = o; o += ((K * 4 + 15) / 16) * 16;
    s.bar_off = o; o += 128;
    s.total = o + 1024;   // slack for the 1024-byte alignment of the base
    return s;
}

// byte offset of element (row, col) inside one swizzled 128-row x 64-col bf16 atom
__device__ __forceinline__ int sw128_off(int row, int col) {
    return row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1));
}

struct Bars {
    uint64_t acc_full[NSTAGE_MAX];    // UMMAs of the stage done + E rows staged   (2 arrivals: commit, issuer)
    uint64_t acc_empty[NSTAGE_MAX];   // every epilogue warp has read the stage's accumulators (EPI_WARPS arrivals)
    uint32_t tmem_base;
    int abort_flag;
    int n_slots;
};

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// SILU is a compile-time switch: a run-time test inside the unrolled epilogue would put a branch between every
// pair of gate elements and stop the scheduler from overlapping their MUFU and FMA latencies.
// ROWS: slot-embedding rows are looked up through FlashArgs::erow (tables shared between samples)
template <bool SILU, int NK, bool ROWS>
__global__ void __launch_bounds__(THREADS, 1) k_flash_fwd_tc(FlashArgs a, int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int N = NK * 64, ldR = N + 4, NSTAGE = nstage(NK);
    const Smem L = smem_layout(N, a.K);
    unsigned char* A_sh = sm + L.a_off;
    unsigned char* B_sh = sm + L.b_off;
    float* R_sh = reinterpret_cast<float*>(sm + L.r_off);
    float* E_sh = reinterpret_cast<float*>(sm + L.e_off);
    unsigned char* ring_sh = sm + L.ring_off;
    __nv_bfloat16* Rb_sh = reinterpret_cast<__nv_bfloat16*>(sm + L.r_off);     // N = 64
    uint32_t* TS2_sh = reinterpret_cast<uint32_t*>(sm + L.ts_off);             // N = 64: packed bf16 pairs
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
        bars->abort_flag = *reinterpret_cast<volatile int*>(status);   // an earlier CTA already gave up: do nothing
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
        // B operand: rows = the pair's 128 output columns, K-major over n; 0.5 * W when the gate is SiLU (the
        // epilogue evaluates SiLU(x) = h + h * tanh(h) with h = x / 2)
        const float wscale = SILU ? 0.5f : 1.0f;
        for (int i = tid; i < N * HPC * HD; i += THREADS) {
            const int n = i / (HPC * HD), dd = i % (HPC * HD);
            const float w = a.W[(size_t)n * D + hp * HPC * HD + dd] * wscale;
            unsigned char* dstw = B_sh + (n >> 6) * ATOM_BYTES + sw128_off(dd, n & 63);
            if (NK == 1) *reinterpret_cast<__half*>(dstw) = __float2half_rn(w * STATE_F16_UNSCALE);   // the state operand carries 1/64
            else *reinterpret_cast<__nv_bfloat16*>(dstw) = __float2bfloat16(w);
        }
        for (int i = tid; i < TM * N; i += THREADS) {   // decay powers rho_n^r, r = 0..127
            const int r = i / N, n = i % N;
            const float pw = exp2f((float)r * log2f(a.rhos[n]));
            if (NK == 1) reinterpret_cast<__half*>(Rb_sh)[r * N + n] = __float2half_rn(pw); else R_sh[r * ldR + n] = pw;
        }
        for (int i = tid; i < TM; i += THREADS) {
            const int tt = t0 + i;
            tok_sh[i] = (tt < Lb) ? (int)(a.x[(size_t)b * a.T + tt] & 0x7fffffffLL) : -1;
        }
        if (NK == 1) {   // restart values of the tile's 128 steps: read from shared memory by the hot rows
            for (int i = tid; i < TM * (N / 4); i += THREADS) {
                const int r = i / (N / 4), c4 = i % (N / 4);
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (t0 + r < a.T) v = __ldg(reinterpret_cast<const float4*>(a.tok_state + ((size_t)b * a.T + t0 + r) * N) + c4);
                const float sc = STATE_F16_SCALE;                           // "+1": the occurrence itself
                TS2_sh[2 * i] = pack_f16x2((v.x + 1.0f) * sc, (v.y + 1.0f) * sc);
                TS2_sh[2 * i + 1] = pack_f16x2((v.z + 1.0f) * sc, (v.w + 1.0f) * sc);
            }
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
        // ============================================================ producer warpgroup: one thread per time step
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        const uint32_t idesc = umma_idesc_16(TM, ACC_COLS, 0, 0, NK == 1 ? 0 : 1, NK == 1 ? 0 : 1);   // N = 64: fp16 operands
        const uint32_t a_base = smem_u32(A_sh), b_base = smem_u32(B_sh);
        const int wi = row >> 5, bi = row & 31;
        const int esize = (a.e_dt == MBEMA_F32) ? 4 : 2;
        const int s_chunks = N / 8, e_chunks = ACC_COLS * esize / 16;     // 16-byte chunks per row (bf16 snapshot; raw E)
        const __nv_bfloat16* snap16 = reinterpret_cast<const __nv_bfloat16*>(a.tile_state + (size_t)a.B * a.nT * a.K * N);
        // Asynchronous prefetch of slot j's snapshot row and raw E_k / E_v rows into ring stage j % RING.
        // E row of the next slot to prefetch (tables shared between samples: one index load per slot, a slot ahead)
        size_t erow_next = (ROWS && n_slots > 0) ? (size_t)a.erow[(size_t)b * a.K + slot_sh[0]] : 0;
        auto prefetch = [&](int j) {
            if (j < n_slots && row < s_chunks + 2 * e_chunks) {   // threads without a chunk to copy skip the address arithmetic too
                const int k = slot_sh[j];
                const size_t er = ROWS ? erow_next : (size_t)b * a.K + k;
                if (ROWS && j + 1 < n_slots) erow_next = (size_t)a.erow[(size_t)b * a.K + slot_sh[j + 1]];
                unsigned char* dst = ring_sh + (j % RING) * RING_STAGE_BYTES;
                const unsigned char* srcS = reinterpret_cast<const unsigned char*>(snap16 + (((size_t)b * a.nT + tile) * a.K + k) * N);
                const size_t eoff = (er * D + hp * ACC_COLS) * esize;
                const unsigned char* srcK = reinterpret_cast<const unsigned char*>(a.Ek) + eoff;
                const unsigned char* srcV = reinterpret_cast<const unsigned char*>(a.Ev) + eoff;
                for (int c = row; c < s_chunks + 2 * e_chunks; c += PROD_THREADS) {
                    const unsigned char* src;
                    unsigned char* d;
                    if (c < s_chunks) { src = srcS + c * 16; d = dst + c * 16; }
                    else if (c < s_chunks + e_chunks) { src = srcK + (c - s_chunks) * 16; d = dst + 512 + (c - s_chunks) * 16; }
                    else { src = srcV + (c - s_chunks - e_chunks) * 16; d = dst + 512 + ACC_COLS * 4 + (c - s_chunks - e_chunks) * 16; }
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(d)), "l"(src) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        // this row's decay powers as packed bf16 pairs (register-resident when N == 64)
        uint32_t R2[NK == 1 ? 32 : 1];
        if (NK == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) R2[j] = *reinterpret_cast<const uint32_t*>(Rb_sh + row * N + 2 * j);
        }
        for (int j = 0; j < PD; ++j) prefetch(j);
        asm volatile("cp.async.wait_group %0;" ::"n"(PD - 1) : "memory");
        named_bar_sync(1, PROD_THREADS);                // slot 0's rows are visible to the whole warpgroup
        for (int i = 0; i < n_slots; ++i) {
            const int st = i % NSTAGE, u = i / NSTAGE;
            prefetch(i + PD);
            asm volatile("cp.async.wait_group %0;" ::"n"(PD - 1) : "memory");   // this thread's copies for slot i+1 landed
            // stage st (A tile, E rows, accumulators) is free once the epilogue of slot i - NSTAGE has finished
            if (i >= NSTAGE) mbar_wait(&bars->acc_empty[st], (uint32_t)((u - 1) & 1), abort_flag);
            const int keyf = key_sh[i];
            const int key = keyf & 0x7fffffff;
            const unsigned char* rg = ring_sh + (i % RING) * RING_STAGE_BYTES;
            // E_k / E_v rows of the slot for the head pair, as fp32: thread p converts column p of both
            {
                float* dst = E_sh + st * 2 * ACC_COLS + row;
                if (esize == 4) {
                    dst[0] = reinterpret_cast<const float*>(rg + 512)[row];
                    dst[ACC_COLS] = reinterpret_cast<const float*>(rg + 512 + ACC_COLS * 4)[row];
                } else {
                    dst[0] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(rg + 512)[row]);
                    dst[ACC_COLS] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(rg + 512 + ACC_COLS * 4)[row]);
                }
            }
            // last occurrence of the slot's token strictly before this row, inside the tile
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
            unsigned char* Arow = A_sh + st * NK * ATOM_BYTES + row * 128;
            if (s >= 0) {   // restart from the token's own state at that occurrence (+1 for the occurrence itself)
                if (NK == 1) {   // bf16 restart value x bf16 power, rounded once more by the packed multiply; the
                                 // backward rebuilds the same tiles with the same operations
                    const uint32_t* tsr = TS2_sh + s * (N / 2);
                    const uint32_t* rr = reinterpret_cast<const uint32_t*>(Rb_sh + (row - s) * N);
#pragma unroll
                    for (int cc = 0; cc < 8; ++cc) {
                        const uint4 tv = *reinterpret_cast<const uint4*>(tsr + 4 * cc);
                        const uint4 rv = *reinterpret_cast<const uint4*>(rr + 4 * cc);
                        uint4 pk;
                        pk.x = mul_f16x2(tv.x, rv.x);
                        pk.y = mul_f16x2(tv.y, rv.y);
                        pk.z = mul_f16x2(tv.z, rv.z);
                        pk.w = mul_f16x2(tv.w, rv.w);
                        *reinterpret_cast<uint4*>(Arow + (((cc & 7) ^ (row & 7)) << 4)) = pk;
                    }
                } else {
                    const float* base = a.tok_state + ((size_t)b * a.T + t0 + s) * N;
                    const float* Rrow = R_sh + (row - s) * ldR;
#pragma unroll 2
                    for (int cc = 0; cc < N / 8; ++cc) {
                        const int n0 = cc * 8;
                        const float4 b0 = __ldg(reinterpret_cast<const float4*>(base + n0));
                        const float4 b1 = __ldg(reinterpret_cast<const float4*>(base + n0 + 4));
                        const float4 r0 = *reinterpret_cast<const float4*>(Rrow + n0);
                        const float4 r1 = *reinterpret_cast<const float4*>(Rrow + n0 + 4);
                        uint4 pk;
                        pk.x = pack_bf16x2(fmaf(b0.x, r0.x, r0.x), fmaf(b0.y, r0.y, r0.y));
                        pk.y = pack_bf16x2(fmaf(b0.z, r0.z, r0.z), fmaf(b0.w, r0.w, r0.w));
                        pk.z = pack_bf16x2(fmaf(b1.x, r1.x, r1.x), fmaf(b1.y, r1.y, r1.y));
                        pk.w = pack_bf16x2(fmaf(b1.z, r1.z, r1.z), fmaf(b1.w, r1.w, r1.w));
                        *reinterpret_cast<uint4*>(Arow + (cc >> 3) * ATOM_BYTES + (((cc & 7) ^ (row & 7)) << 4)) = pk;
                    }
                }
            } else {        // plain decay of the tile-start snapshot: bf16 snapshot (prefetched, broadcast reads) times
                            // this row's decay powers; product rounded to bf16 by the packed multiply
                if (NK == 1) {
#pragma unroll
                    for (int cc = 0; cc < 8; ++cc) {
                        const uint4 sv = *reinterpret_cast<const uint4*>(rg + cc * 16);
                        uint4 pk;
                        pk.x = mul_f16x2(sv.x, R2[4 * cc]);
                        pk.y = mul_f16x2(sv.y, R2[4 * cc + 1]);
                        pk.z = mul_f16x2(sv.z, R2[4 * cc + 2]);
                        pk.w = mul_f16x2(sv.w, R2[4 * cc + 3]);
                        *reinterpret_cast<uint4*>(Arow + (((cc & 7) ^ (row & 7)) << 4)) = pk;
                    }
                } else {
                    const float* Rrow = R_sh + row * ldR;
#pragma unroll 2
                    for (int cc = 0; cc < N / 8; ++cc) {
                        const int n0 = cc * 8;
                        const uint4 sv = *reinterpret_cast<const uint4*>(rg + cc * 16);
                        const float4 r0 = *reinterpret_cast<const float4*>(Rrow + n0);
                        const float4 r1 = *reinterpret_cast<const float4*>(Rrow + n0 + 4);
                        uint4 pk;
                        pk.x = pack_bf16x2(bf16_lo(sv.x) * r0.x, bf16_hi(sv.x) * r0.y);
                        pk.y = pack_bf16x2(bf16_lo(sv.y) * r0.z, bf16_hi(sv.y) * r0.w);
                        pk.z = pack_bf16x2(bf16_lo(sv.z) * r1.x, bf16_hi(sv.z) * r1.y);
                        pk.w = pack_bf16x2(bf16_lo(sv.w) * r1.z, bf16_hi(sv.w) * r1.w);
                        *reinterpret_cast<uint4*>(Arow + (cc >> 3) * ATOM_BYTES + (((cc & 7) ^ (row & 7)) << 4)) = pk;
                    }
                }
            }
            fence_proxy_async_smem();
            named_bar_sync(1, PROD_THREADS);          // the whole tile and both E rows are in shared memory
            if (warp == EPI_WARPS + (i & 3) && lane == 0) {   // one thread issues the UMMAs of this slot (the role rotates)
                tc_fence_after_sync();
                for (int atom = 0; atom < NK; ++atom) {
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16) {
                        const uint64_t adesc = umma_desc_k_sw128(a_base + (st * NK + atom) * ATOM_BYTES + k16 * 32);
                        const uint64_t bdesc = umma_desc_k_sw128(b_base + atom * ATOM_BYTES + k16 * 32);
                        umma_bf16_ss(tmem_base + (uint32_t)(st * ACC_COLS), adesc, bdesc, idesc, (atom | k16) != 0 ? 1u : 0u);
                    }
                }
                umma_commit(&bars->acc_full[st]);   // first arrival: the UMMAs above have completed
                mbar_arrive(&bars->acc_full[st]);   // second arrival: releases the staged E rows
            }
        }
    } else {
        // ============================================================ epilogue warpgroups: a thread per time step, a head per warpgroup
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int wg = warp >> 2;
        const int h = hp * HPC + wg;
        const size_t qoff = (((size_t)b * a.H + h) * a.T + t) * HD;
        const bool row_ok = t < Lb;
        float q[HD], o[HD];
#pragma unroll
        for (int i = 0; i < HD; i += 4) {
            float4 v = row_ok ? ld4_dyn_f32(a.Q, a.q_dt, qoff + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            q[i] = v.x * 0.125f; q[i + 1] = v.y * 0.125f; q[i + 2] = v.z * 0.125f; q[i + 3] = v.w * 0.125f;
            o[i] = o[i + 1] = o[i + 2] = o[i + 3] = 0.f;
        }
        const float rest = a.v_total - (float)a.kcount[b];
        float m, l;
        if (!a.listed_only && rest > 0.f) { m = 0.f; l = rest; } else { m = -INFINITY; l = 0.f; }
        const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(wg * HD);

        for (int i = 0; i < n_slots; ++i) {
            const int st = i % NSTAGE, u = i / NSTAGE;
            mbar_wait(&bars->acc_full[st], (uint32_t)(u & 1), abort_flag);
            tc_fence_after_sync();
            float pre[HD];
            tmem_ld_32x32b_x32(t_lane + st * ACC_COLS, pre);
            tmem_ld_32x32b_x32(t_lane + st * ACC_COLS + 32, pre + 32);
            tmem_wait_ld();

            const float* ek = E_sh + st * 2 * ACC_COLS + wg * HD;
            const float* ev = ek + ACC_COLS;
            float sp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < HD; j += 4) {
                const float4 e = *reinterpret_cast<const float4*>(ek + j);
                const float ee[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const float hh = pre[j + v];
                    const float g = SILU ? fmaf(hh, tanh_approx(hh), hh) : hh;
                    pre[j + v] = g;
                    sp[v] = fmaf(g * q[j + v], ee[v], sp[v]);
                }
            }
            const float s = (sp[0] + sp[1]) + (sp[2] + sp[3]);
            const float m_new = fmaxf(m, s);
            if (m_new > m) {
                const float alpha = __expf(m - m_new);
                l *= alpha;
#pragma unroll
                for (int j = 0; j < HD; ++j) o[j] *= alpha;
                m = m_new;
            }
            const float p = __expf(s - m);
            l += p;
#pragma unroll
            for (int j = 0; j < HD; j += 4) {
                const float4 e = *reinterpret_cast<const float4*>(ev + j);
                o[j] = fmaf(p * pre[j], e.x, o[j]);
                o[j + 1] = fmaf(p * pre[j + 1], e.y, o[j + 1]);
                o[j + 2] = fmaf(p * pre[j + 2], e.z, o[j + 2]);
                o[j + 3] = fmaf(p * pre[j + 3], e.w, o[j + 3]);
            }
            // accumulators and E rows of this stage are consumed
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->acc_empty[st]);
        }
        if (t < a.T) {
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
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (tid == 0 && bars->abort_flag) atomicExch(status, 1);   // sticky: later CTAs of this launch skip their work
}

}  // namespace tc

bool flash_tc_supported(int H, int N, int K) { return (H % tc::HPC) == 0 && (N == 64 || N == 128) && K <= tc::MAX_SLOTS; }

size_t flash_fwd_tc_ws() { return 256; }

int flash_fwd_tc(const FlashArgs& a, void* ws, cudaStream_t st) {
    int* status = reinterpret_cast<int*>((reinterpret_cast<uintptr_t>(ws) + 15) & ~uintptr_t(15));
    MBEMA_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int), st));
    const tc::Smem L = tc::smem_layout(a.N, a.K);
    if (L.total > 227 * 1024) return MBEMA_ERR_UNSUPPORTED;
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
