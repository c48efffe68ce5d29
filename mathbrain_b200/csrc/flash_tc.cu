// Flash-EMA gated cross-attention on the Blackwell tensor cores (MBEMA_MODE_TC_BF16), forward.
//
// One CTA owns (sample b, a 128-step time tile, a pair of heads) and loops over the sample's valid slots.
// For slot k the 128 x N state tile A[t, :] = M_t[k, :] (bf16, 128-byte-swizzled K-major rows) is rebuilt in
// shared memory from the tile-start snapshot and a table of decay powers; one elected thread issues
//     pre[128 x 128] = A[128 x N] @ (W_pe[:, 2 heads])            tcgen05.mma, fp32 accumulators in TMEM
// and the eight warps (a warpgroup per head; a thread per time step) read their 64 accumulator columns with
// tcgen05.ld and fuse SiLU, K = E_k*gate, V = E_v*gate, the score, the online softmax and the P.V update, all
// thread-local.  A tiles and TMEM accumulators are double buffered: while the epilogue of slot i runs, the
// tensor core already works on slot i+1.  Hand-offs go through mbarriers with bounded waits.
// The CTA has exactly 8 warps (registers are allocated to warps in groups of four, and a thread needs ~230 of
// them for q, the output row and 64 accumulator columns); thread 0 doubles as the UMMA issuer.
#include "flash.cuh"
#include "sm100_ptx.cuh"

namespace mbema {
namespace tc {

using namespace ptx;

static constexpr int TM = MBEMA_TILE_T;        // rows (time steps) per CTA
static constexpr int HPC = 2;                  // heads per CTA
static constexpr int HD = 64;
static constexpr int EPI_WARPS = 4 * HPC;
static constexpr int EPI_THREADS = 32 * EPI_WARPS;
static constexpr int THREADS = EPI_THREADS;
static constexpr int ATOM_BYTES = TM * 128;        // one 128-row x 64-column bf16 swizzle atom
static constexpr int E_STAGES = 8;                 // slot-embedding rows staged ahead (warps drift up to 4 slots apart)
static constexpr int TMEM_COLS = 2 * HPC * HD;     // two accumulator buffers of HPC*64 fp32 columns
static constexpr int MAX_SLOTS = 16384;

struct Smem {
    // offsets (bytes) into the dynamic shared memory block, base aligned to 1024
    int a_off, b_off, r_off, e_off, tok_off, slot_off, bar_off, total;
};

__host__ __device__ inline Smem smem_layout(int N, int K) {
    const int NK = N / 64;
    Smem s;
    int o = 0;
    s.a_off = o; o += 2 * NK * ATOM_BYTES;
    s.b_off = o; o += NK * ATOM_BYTES;
    s.r_off = o; o += TM * (N + 4) * 4;
    s.e_off = o; o += E_STAGES * 2 * HPC * HD * 4;
    s.tok_off = o; o += TM * 4;
    s.slot_off = o; o += ((K * 2 + 15) / 16) * 16;
    s.bar_off = o; o += 128;
    s.total = o + 1024;   // slack for the 1024-byte alignment of the base
    return s;
}

// byte offset of element (row, col) inside one swizzled 128-row x 64-col bf16 atom
__device__ __forceinline__ int sw128_off(int row, int col) {
    return row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1));
}

struct Bars {
    uint64_t a_full[2];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    int n_slots;
};

__global__ void __launch_bounds__(THREADS, 1) k_flash_fwd_tc(FlashArgs a, int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int N = a.N, NK = N / 64, ldR = N + 4;
    const Smem L = smem_layout(N, a.K);
    unsigned char* A_sh = sm + L.a_off;
    unsigned char* B_sh = sm + L.b_off;
    float* R_sh = reinterpret_cast<float*>(sm + L.r_off);
    float* E_sh = reinterpret_cast<float*>(sm + L.e_off);
    int* tok_sh = reinterpret_cast<int*>(sm + L.tok_off);
    unsigned short* slot_sh = reinterpret_cast<unsigned short*>(sm + L.slot_off);
    Bars* bars = reinterpret_cast<Bars*>(sm + L.bar_off);
    volatile int* abort_flag = &bars->abort_flag;

    const int tile = blockIdx.x, hp = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int D = a.H * HD;
    const int t0 = tile * TM;
    const int Lb = a.seq_lens ? min(max(a.seq_lens[b], 0), a.T) : a.T;
    const int wg = warp >> 2;                       // head within the pair (epilogue warps)
    const int row = (warp & 3) * 32 + lane;         // time step within the tile == TMEM lane
    const int h = hp * HPC + wg;
    const int t = t0 + row;
    const size_t qoff = (((size_t)b * a.H + h) * a.T + t) * HD;

    if (t0 >= Lb) {   // whole tile beyond the valid length: define the outputs and leave (uniform per CTA)
        if (t < a.T) {
#pragma unroll
            for (int i = 0; i < HD; i += 4) *reinterpret_cast<float4*>(a.O + qoff + i) = make_float4(0.f, 0.f, 0.f, 0.f);
            a.LSE[((size_t)b * a.H + h) * a.T + t] = 0.f;
        }
        return;
    }

    // ---------------------------------------------------------------- prologue
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->a_full[i], EPI_WARPS);
            mbar_init(&bars->acc_full[i], 2);
            mbar_init(&bars->acc_empty[i], EPI_WARPS);
        }
        bars->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc(&bars->tmem_base, TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == 1) {
        // ordered compaction of the valid slot indices
        int n = 0;
        for (int k0 = 0; k0 < a.K; k0 += 32) {
            const int k = k0 + lane;
            const bool ok = (k < a.K) && (a.unique[(size_t)b * a.K + k] >= 0);
            const unsigned m = __ballot_sync(0xffffffffu, ok);
            if (ok) slot_sh[n + __popc(m & ((1u << lane) - 1u))] = (unsigned short)k;
            n += __popc(m);
        }
        if (lane == 0) bars->n_slots = n;
    }
    // B operand: rows = the pair's 128 output columns, K-major over n; 0.5 * W when the gate is SiLU (the
    // epilogue evaluates SiLU(x) = h + h * tanh(h) with h = x / 2)
    {
        const float wscale = a.silu ? 0.5f : 1.0f;
        for (int i = tid; i < N * HPC * HD; i += THREADS) {
            const int n = i / (HPC * HD), dd = i % (HPC * HD);
            const float w = a.W[(size_t)n * D + hp * HPC * HD + dd] * wscale;
            *reinterpret_cast<__nv_bfloat16*>(B_sh + (n >> 6) * ATOM_BYTES + sw128_off(dd, n & 63)) = __float2bfloat16(w);
        }
        for (int i = tid; i < TM * N; i += THREADS) {
            const int r = i / N, n = i % N;
            R_sh[r * ldR + n] = exp2f((float)r * log2f(a.rhos[n]));
        }
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
    const int n_slots = bars->n_slots;

    // ---------------------------------------------------------------- per-thread state: one time step of one head
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
    const int cc0 = wg * (N / (8 * HPC)), cc1 = cc0 + N / (8 * HPC);   // this warpgroup's 16-byte chunks of a row
    const uint32_t idesc = umma_idesc_bf16(TM, HPC * HD, 0, 0);
    const uint32_t a_base = smem_u32(A_sh), b_base = smem_u32(B_sh);

    // Stage slot i: this thread's share of the bf16 state tile A (rows = time steps) and of the slot's E_k / E_v
    // rows (converted to fp32), then signal "A full".
    auto stage_slot = [&](int i) {
        const int k = slot_sh[i];
        const int key = (int)(a.unique[(size_t)b * a.K + k] & 0x7fffffffLL);
        {
            const int which = tid >> 7, col = tid & 127;     // 0: E_k, 1: E_v; column within the head pair
            const float v = ld_dyn_f32(which ? a.Ev : a.Ek, a.e_dt, ((size_t)b * a.K + k) * D + hp * HPC * HD + col);
            E_sh[((i % E_STAGES) * 2 + which) * HPC * HD + col] = v;
        }
        unsigned w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = __ballot_sync(0xffffffffu, tok_sh[32 * j + lane] == key);
        const int wi = row >> 5, bi = row & 31;
        int s = -1;
#pragma unroll
        for (int j = 3; j >= 0; --j) {
            unsigned mm = (j > wi) ? 0u : (j == wi ? (w[j] & ((1u << bi) - 1u)) : w[j]);
            if (s < 0 && mm) s = j * 32 + 31 - __clz(mm);
        }
        const float* base;
        float add;
        int rr;
        if (s >= 0) {   // restart from the token's own state at its last occurrence inside the tile
            base = a.tok_state + ((size_t)b * a.T + t0 + s) * N;
            add = 1.0f;
            rr = row - s;
        } else {        // plain decay of the tile-start snapshot
            base = a.tile_state + (((size_t)b * a.nT + tile) * a.K + k) * N;
            add = 0.0f;
            rr = row;
        }
        const float* Rrow = R_sh + rr * ldR;
        unsigned char* Abuf = A_sh + (i & 1) * NK * ATOM_BYTES;
        for (int cc = cc0; cc < cc1; ++cc) {
            const int n0 = cc * 8;
            const float4 b0 = __ldg(reinterpret_cast<const float4*>(base + n0));
            const float4 b1 = __ldg(reinterpret_cast<const float4*>(base + n0 + 4));
            const float4 r0 = *reinterpret_cast<const float4*>(Rrow + n0);
            const float4 r1 = *reinterpret_cast<const float4*>(Rrow + n0 + 4);
            uint4 pk;
            pk.x = pack_bf16x2((b0.x + add) * r0.x, (b0.y + add) * r0.y);
            pk.y = pack_bf16x2((b0.z + add) * r0.z, (b0.w + add) * r0.w);
            pk.z = pack_bf16x2((b1.x + add) * r1.x, (b1.y + add) * r1.y);
            pk.w = pack_bf16x2((b1.z + add) * r1.z, (b1.w + add) * r1.w);
            *reinterpret_cast<uint4*>(Abuf + (cc >> 3) * ATOM_BYTES + row * 128 + (((cc & 7) ^ (row & 7)) << 4)) = pk;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->a_full[i & 1]);
    };

    // Thread 0 only: once every warp has staged slot i (and the accumulator buffer is free), issue its UMMAs.
    auto issue_slot = [&](int i) {
        const int buf = i & 1, u = i >> 1;
        mbar_wait(&bars->a_full[buf], (uint32_t)(u & 1), abort_flag);
        if (i >= 2) mbar_wait(&bars->acc_empty[buf], (uint32_t)((u - 1) & 1), abort_flag);
        tc_fence_after_sync();
        for (int atom = 0; atom < NK; ++atom) {
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16) {
                const uint64_t adesc = umma_desc_k_sw128(a_base + (buf * NK + atom) * ATOM_BYTES + k16 * 32);
                const uint64_t bdesc = umma_desc_k_sw128(b_base + atom * ATOM_BYTES + k16 * 32);
                umma_bf16_ss(tmem_base + (uint32_t)(buf * HPC * HD), adesc, bdesc, idesc, (atom | k16) != 0 ? 1u : 0u);
            }
        }
        umma_commit(&bars->acc_full[buf]);   // first arrival: the UMMAs above have completed
        mbar_arrive(&bars->acc_full[buf]);   // second arrival: releases the staged E rows seen through a_full
    };

    if (n_slots > 0) {
        stage_slot(0);
        if (tid == 0) issue_slot(0);
    }
    for (int i = 0; i < n_slots; ++i) {
        if (i + 1 < n_slots) {
            stage_slot(i + 1);
            if (tid == 0) issue_slot(i + 1);
            __syncwarp();
        }
        const int buf = i & 1;
        mbar_wait(&bars->acc_full[buf], (uint32_t)((i >> 1) & 1), abort_flag);
        tc_fence_after_sync();
        float pre[HD];
        const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(buf * HPC * HD + wg * HD);
        tmem_ld_32x32b_x32(taddr, pre);
        tmem_ld_32x32b_x32(taddr + 32, pre + 32);
        tmem_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->acc_empty[buf]);

        const float* ek = E_sh + ((i % E_STAGES) * 2 + 0) * HPC * HD + wg * HD;
        const float* ev = ek + HPC * HD;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < HD; j += 4) {
            const float4 e = *reinterpret_cast<const float4*>(ek + j);
            const float ee[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float hh = pre[j + u];
                const float g = a.silu ? fmaf(hh, tanh_approx(hh), hh) : hh;
                pre[j + u] = g;
                s = fmaf(g * q[j + u], ee[u], s);
            }
        }
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
    }
    if (t < a.T) {
        const float inv = (row_ok && l > 0.f) ? 1.0f / l : 0.f;
#pragma unroll
        for (int i = 0; i < HD; i += 4)
            *reinterpret_cast<float4*>(a.O + qoff + i) = make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
        a.LSE[((size_t)b * a.H + h) * a.T + t] = (row_ok && l > 0.f) ? m + logf(l) : 0.f;
    }
    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (tid == 0 && bars->abort_flag) atomicExch(status, 1);
}

}  // namespace tc

bool flash_tc_supported(int H, int N, int K) { return (H % tc::HPC) == 0 && (N == 64 || N == 128) && K <= tc::MAX_SLOTS; }

size_t flash_fwd_tc_ws() { return 256; }

int flash_fwd_tc(const FlashArgs& a, void* ws, cudaStream_t st) {
    int* status = reinterpret_cast<int*>((reinterpret_cast<uintptr_t>(ws) + 15) & ~uintptr_t(15));
    MBEMA_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int), st));
    const tc::Smem L = tc::smem_layout(a.N, a.K);
    MBEMA_CUDA_TRY(cudaFuncSetAttribute(tc::k_flash_fwd_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total));
    dim3 grid(a.nT, a.H / tc::HPC, a.B);
    tc::k_flash_fwd_tc<<<grid, tc::THREADS, L.total, st>>>(a, status);
    return check_launch();
}

}  // namespace mbema
