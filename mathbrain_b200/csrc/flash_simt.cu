// Flash-EMA gated cross-attention, fp32 arithmetic on the CUDA cores (MBEMA_MODE_FP32).
//
// Work decomposition (shared with the tensor-core path): one CTA owns (sample b, head h, a block of
// consecutive time steps) and loops over the sample's listed slots.  A thread owns one time step (row) and
// 16 of the head's 64 columns, so the online softmax, the output accumulator and dQ are thread-local and the
// only cross-thread traffic in the forward is a 4-lane shuffle for the score.
//
// For slot k the rows of the state matrix A[t, :] = M_t[k, :] are rebuilt from the tile-start snapshot
// (row t of tile: snapshot * rho^(t - t0)); rows that follow an occurrence of the slot's token inside the
// tile restart from the token's own state at that occurrence (+1), found with warp ballots over the tile's
// tokens.  pre = A @ W_pe[:, head], gate = SiLU(pre), K = E_k * gate, V = E_v * gate.
#include "flash.cuh"

namespace mbema {

static constexpr int FS_ROWS = 64;           // time steps per CTA (half a snapshot tile)
static constexpr int FS_THREADS = FS_ROWS * 4;
static constexpr int FS_HD = 64;
static constexpr int FS_ZLD = 72;            // padded row length of the backward staging tiles

__device__ __forceinline__ int zcol(int c) { return c + ((c >> 5) << 2); }
// shared-memory regions start on 16-byte boundaries (float4 accesses) for every N
__host__ __device__ inline int round4(int v) { return (v + 3) & ~3; }


// Row state source for slot `key`: returns the step offset s (within the tile) of the last occurrence of the
// slot's token strictly before row r, or -1.
__device__ __forceinline__ int last_occurrence_before(const int* tok_sh, int key, int r, int lane) {
    unsigned w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = __ballot_sync(0xffffffffu, tok_sh[32 * j + lane] == key);
    const int wi = r >> 5, bi = r & 31;
    int s = -1;
#pragma unroll
    for (int j = 3; j >= 0; --j) {
        unsigned m = (j > wi) ? 0u : (j == wi ? (w[j] & ((1u << bi) - 1u)) : w[j]);
        if (s < 0 && m) s = j * 32 + 31 - __clz(m);
    }
    return s;
}

// Shared prologue: builds A rows for slot k into A_sh (each thread fills columns dg, dg+4, ...)
__device__ __forceinline__ void build_state_rows(const FlashArgs& a, int b, int tile, int k, int key, int r_tile,
                                                 int tr, int dg, int lane, const int* tok_sh, const float* l2r_sh,
                                                 float* A_sh, int ldA) {
    const int s = last_occurrence_before(tok_sh, key, r_tile, lane);
    const float* base;
    float add, dt;
    if (s >= 0) {
        base = a.tok_state + ((size_t)b * a.T + (size_t)tile * MBEMA_TILE_T + s) * a.N;
        add = 1.0f;
        dt = (float)(r_tile - s);
    } else {
        base = a.tile_state + (((size_t)b * a.nT + tile) * a.K + k) * a.N;
        add = 0.0f;
        dt = (float)r_tile;
    }
    for (int n = dg; n < a.N; n += 4) A_sh[tr * ldA + n] = (base[n] + add) * exp2f(dt * l2r_sh[n]);
}

// ------------------------------------------------------------------------------------------------
// forward
// dynamic smem: W_sh[N][64] | A_sh[FS_ROWS][N+1] | l2r_sh[N] | tok_sh[128]
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(FS_THREADS) k_flash_fwd_simt(FlashArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int N = a.N, ldA = N + 1;
    float* W_sh = smem;
    float* A_sh = W_sh + N * FS_HD;
    float* l2r_sh = A_sh + round4(FS_ROWS * ldA);
    int* tok_sh = reinterpret_cast<int*>(l2r_sh + round4(N));

    const int half = blockIdx.x & 1, tile = blockIdx.x >> 1;
    const int h = blockIdx.y, b = a.order ? a.order[blockIdx.z] : (int)blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31;
    const int tr = tid >> 2, dg = tid & 3;
    const int D = a.H * FS_HD;
    const int t0 = tile * MBEMA_TILE_T;
    const int r_tile = half * FS_ROWS + tr;   // row index inside the snapshot tile
    const int t = t0 + r_tile;
    const int Lb = a.seq_lens ? min(max(a.seq_lens[b], 0), a.T) : a.T;
    const int row0 = t0 + half * FS_ROWS;
    if (row0 >= a.T) return;
    const bool row_ok = t < Lb;
    const size_t qoff = (((size_t)b * a.H + h) * a.T + t) * FS_HD + dg * 16;
    if (row0 >= Lb) {  // nothing to compute: define the skipped outputs
        if (t < a.T) {
#pragma unroll
            for (int i = 0; i < 16; i += 4) *reinterpret_cast<float4*>(a.O + qoff + i) = make_float4(0.f, 0.f, 0.f, 0.f);
            if (dg == 0) a.LSE[((size_t)b * a.H + h) * a.T + t] = 0.f;
        }
        return;
    }
    for (int i = tid; i < N * FS_HD; i += FS_THREADS) W_sh[i] = a.W[(size_t)(i / FS_HD) * D + h * FS_HD + (i % FS_HD)];
    for (int i = tid; i < N; i += FS_THREADS) l2r_sh[i] = log2f(a.rhos[i]);
    for (int i = tid; i < MBEMA_TILE_T; i += FS_THREADS) {
        const int tt = t0 + i;
        tok_sh[i] = (tt < Lb) ? (int)(a.x[(size_t)b * a.T + tt] & 0x7fffffffLL) : -1;
    }
    const float scale = 0.125f;  // 1/sqrt(64)
    float q[16], o[16];
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
        float4 v = row_ok ? ld4_dyn_f32(a.Q, a.q_dt, qoff + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        q[i] = v.x * scale; q[i + 1] = v.y * scale; q[i + 2] = v.z * scale; q[i + 3] = v.w * scale;
        o[i] = o[i + 1] = o[i + 2] = o[i + 3] = 0.f;
    }
    const int kb = a.kcount[b];
    const float rest = a.v_total - (float)kb;
    float m, l;
    if (!a.listed_only && rest > 0.f) { m = 0.f; l = rest; } else { m = -INFINITY; l = 0.f; }
    __syncthreads();

    for (int k = 0; k < a.K; ++k) {
        const long long kv = a.unique[(size_t)b * a.K + k];
        if (kv < 0) continue;  // uniform across the CTA
        const int key = (int)(kv & 0x7fffffffLL);
        build_state_rows(a, b, tile, k, key, r_tile, tr, dg, lane, tok_sh, l2r_sh, A_sh, ldA);
        const size_t eoff = e_row(a, b, k) * D + h * FS_HD + dg * 16;
        float ek[16], ev[16];
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
            float4 v1 = ld4_dyn_f32(a.Ek, a.e_dt, eoff + i);
            float4 v2 = ld4_dyn_f32(a.Ev, a.e_dt, eoff + i);
            ek[i] = v1.x; ek[i + 1] = v1.y; ek[i + 2] = v1.z; ek[i + 3] = v1.w;
            ev[i] = v2.x; ev[i + 1] = v2.y; ev[i + 2] = v2.z; ev[i + 3] = v2.w;
        }
        __syncthreads();
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
        const float* arow = A_sh + tr * ldA;
        const float* wcol = W_sh + dg * 16;
#pragma unroll 4
        for (int n = 0; n < N; ++n) {
            const float av = arow[n];
            const float4* wp = reinterpret_cast<const float4*>(wcol + n * FS_HD);
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
        const float m_new = fmaxf(m, part);
        const float alpha = __expf(m - m_new);
        const float p = __expf(part - m_new);
        l = l * alpha + p;
        m = m_new;
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = fmaf(p, acc[i] * ev[i], o[i] * alpha);
        __syncthreads();
    }
    if (t < a.T) {
        const float inv = (row_ok && l > 0.f) ? 1.0f / l : 0.f;
#pragma unroll
        for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<float4*>(a.O + qoff + i) = make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
        if (dg == 0) a.LSE[((size_t)b * a.H + h) * a.T + t] = (row_ok && l > 0.f) ? m + logf(l) : 0.f;
    }
}

// ------------------------------------------------------------------------------------------------
// backward
// dynamic smem: W_sh[N][64] | A_sh[FS_ROWS][N+1] | l2r_sh[N] | tok_sh[128] | Zk,Zv,Zp [FS_ROWS][FS_ZLD]
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(FS_THREADS) k_flash_bwd_simt(FlashArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int N = a.N, ldA = N + 1;
    float* W_sh = smem;
    float* A_sh = W_sh + N * FS_HD;
    float* l2r_sh = A_sh + round4(FS_ROWS * ldA);
    int* tok_sh = reinterpret_cast<int*>(l2r_sh + round4(N));
    float* Zk = reinterpret_cast<float*>(tok_sh + MBEMA_TILE_T);
    float* Zv = Zk + FS_ROWS * FS_ZLD;
    float* Zp = Zv + FS_ROWS * FS_ZLD;

    const int half = blockIdx.x & 1, tile = blockIdx.x >> 1;
    const int h = blockIdx.y, b = a.order ? a.order[blockIdx.z] : (int)blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31;
    const int tr = tid >> 2, dg = tid & 3;
    const int D = a.H * FS_HD;
    const int t0 = tile * MBEMA_TILE_T;
    const int r_tile = half * FS_ROWS + tr;
    const int t = t0 + r_tile;
    const int Lb = a.seq_lens ? min(max(a.seq_lens[b], 0), a.T) : a.T;
    const int row0 = t0 + half * FS_ROWS;
    // dW mapping: rows n = (tid >> 3) + 32 j, columns (tid & 7) * 8 .. +7
    const int wn = tid >> 3, wd = (tid & 7) * 8;
    float dw[4][8];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) dw[j][i] = 0.f;
    const size_t cta = ((size_t)b * a.H + h) * gridDim.x + blockIdx.x;
    float* part_out = a.dW_part + cta * (size_t)N * FS_HD;

    const bool active = row0 < a.T && row0 < Lb;
    const bool row_ok = t < Lb;
    const size_t qoff = (((size_t)b * a.H + h) * a.T + t) * FS_HD + dg * 16;
    if (!active) {
        if (row0 < a.T && t < a.T) {
#pragma unroll
            for (int i = 0; i < 16; i += 4) *reinterpret_cast<float4*>(a.dQ + qoff + i) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int j = 0; j < 4; ++j)
            if (wn + 32 * j < N)
                for (int i = 0; i < 8; ++i) part_out[(size_t)(wn + 32 * j) * FS_HD + wd + i] = 0.f;
        return;
    }
    for (int i = tid; i < N * FS_HD; i += FS_THREADS) W_sh[i] = a.W[(size_t)(i / FS_HD) * D + h * FS_HD + (i % FS_HD)];
    for (int i = tid; i < N; i += FS_THREADS) l2r_sh[i] = log2f(a.rhos[i]);
    for (int i = tid; i < MBEMA_TILE_T; i += FS_THREADS) {
        const int tt = t0 + i;
        tok_sh[i] = (tt < Lb) ? (int)(a.x[(size_t)b * a.T + tt] & 0x7fffffffLL) : -1;
    }
    const float scale = 0.125f;
    float q[16], dov[16], dq[16];
    float drow = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
        float4 v = row_ok ? ld4_dyn_f32(a.Q, a.q_dt, qoff + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 g = row_ok ? ld4_dyn_f32(a.dO, a.do_dt, qoff + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 ov = row_ok ? *reinterpret_cast<const float4*>(a.O + qoff + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        q[i] = v.x; q[i + 1] = v.y; q[i + 2] = v.z; q[i + 3] = v.w;
        dov[i] = g.x; dov[i + 1] = g.y; dov[i + 2] = g.z; dov[i + 3] = g.w;
        drow += g.x * ov.x + g.y * ov.y + g.z * ov.z + g.w * ov.w;
        dq[i] = dq[i + 1] = dq[i + 2] = dq[i + 3] = 0.f;
    }
    drow += __shfl_xor_sync(0xffffffffu, drow, 1);
    drow += __shfl_xor_sync(0xffffffffu, drow, 2);
    const float lse = row_ok ? a.LSE[((size_t)b * a.H + h) * a.T + t] : 0.f;
    __syncthreads();

    for (int k = 0; k < a.K; ++k) {
        const long long kv = a.unique[(size_t)b * a.K + k];
        if (kv < 0) continue;
        const int key = (int)(kv & 0x7fffffffLL);
        build_state_rows(a, b, tile, k, key, r_tile, tr, dg, lane, tok_sh, l2r_sh, A_sh, ldA);
        const size_t eoff = e_row(a, b, k) * D + h * FS_HD + dg * 16;
        float ek[16], ev[16];
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
            float4 v1 = ld4_dyn_f32(a.Ek, a.e_dt, eoff + i);
            float4 v2 = ld4_dyn_f32(a.Ev, a.e_dt, eoff + i);
            ek[i] = v1.x; ek[i + 1] = v1.y; ek[i + 2] = v1.z; ek[i + 3] = v1.w;
            ev[i] = v2.x; ev[i + 1] = v2.y; ev[i + 2] = v2.z; ev[i + 3] = v2.w;
        }
        __syncthreads();   // A_sh ready; previous slot's Z tiles fully consumed
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
        const float* arow = A_sh + tr * ldA;
        const float* wcol = W_sh + dg * 16;
#pragma unroll 4
        for (int n = 0; n < N; ++n) {
            const float av = arow[n];
            const float4* wp = reinterpret_cast<const float4*>(wcol + n * FS_HD);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float4 wv = wp[j];
                acc[4 * j] = fmaf(av, wv.x, acc[4 * j]);
                acc[4 * j + 1] = fmaf(av, wv.y, acc[4 * j + 1]);
                acc[4 * j + 2] = fmaf(av, wv.z, acc[4 * j + 2]);
                acc[4 * j + 3] = fmaf(av, wv.w, acc[4 * j + 3]);
            }
        }
        // gate, score, dp
        float g[16], dsl[16];
        float sp = 0.f, dpp = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (a.silu) {
                const float sg = sigmoidf_(acc[i]);
                g[i] = acc[i] * sg;
                dsl[i] = sg * (1.0f + acc[i] * (1.0f - sg));
            } else {
                g[i] = acc[i];
                dsl[i] = 1.0f;
            }
            sp = fmaf(g[i] * q[i], ek[i], sp);
            dpp = fmaf(g[i] * dov[i], ev[i], dpp);
        }
        sp += __shfl_xor_sync(0xffffffffu, sp, 1);
        sp += __shfl_xor_sync(0xffffffffu, sp, 2);
        dpp += __shfl_xor_sync(0xffffffffu, dpp, 1);
        dpp += __shfl_xor_sync(0xffffffffu, dpp, 2);
        const float p = row_ok ? __expf(sp * scale - lse) : 0.f;
        const float ds = p * (dpp - drow) * scale;   // d loss / d (q . k) including the 1/sqrt(hd) factor
        float zk[16], zv[16], zp[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            dq[i] = fmaf(ds * ek[i], g[i], dq[i]);
            zk[i] = ds * q[i] * g[i];
            zv[i] = p * dov[i] * g[i];
            zp[i] = (ds * q[i] * ek[i] + p * dov[i] * ev[i]) * dsl[i];
        }
        {
            const int c0 = zcol(dg * 16);
            float* pk = Zk + tr * FS_ZLD + c0;
            float* pv = Zv + tr * FS_ZLD + c0;
            float* pp = Zp + tr * FS_ZLD + c0;
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
                *reinterpret_cast<float4*>(pk + i) = make_float4(zk[i], zk[i + 1], zk[i + 2], zk[i + 3]);
                *reinterpret_cast<float4*>(pv + i) = make_float4(zv[i], zv[i + 1], zv[i + 2], zv[i + 3]);
                *reinterpret_cast<float4*>(pp + i) = make_float4(zp[i], zp[i + 1], zp[i + 2], zp[i + 3]);
            }
        }
        __syncthreads();
        // dW[n, d] += sum_rows A[row, n] * dpre[row, d]
        {
            const int c0 = zcol(wd);
#pragma unroll 2
            for (int r = 0; r < FS_ROWS; ++r) {
                const float4 z0 = *reinterpret_cast<const float4*>(Zp + r * FS_ZLD + c0);
                const float4 z1 = *reinterpret_cast<const float4*>(Zp + r * FS_ZLD + c0 + 4);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (wn + 32 * j < N) {
                        const float av = A_sh[r * ldA + wn + 32 * j];
                        dw[j][0] = fmaf(av, z0.x, dw[j][0]); dw[j][1] = fmaf(av, z0.y, dw[j][1]);
                        dw[j][2] = fmaf(av, z0.z, dw[j][2]); dw[j][3] = fmaf(av, z0.w, dw[j][3]);
                        dw[j][4] = fmaf(av, z1.x, dw[j][4]); dw[j][5] = fmaf(av, z1.y, dw[j][5]);
                        dw[j][6] = fmaf(av, z1.z, dw[j][6]); dw[j][7] = fmaf(av, z1.w, dw[j][7]);
                    }
                }
            }
        }
        // dE_k[k, :], dE_v[k, :]: column sums over the rows of this CTA
        if (tid < 2 * FS_HD) {
            const float* Z = (tid < FS_HD) ? Zk : Zv;
            const int c = tid & (FS_HD - 1);
            const int cc = zcol(c);
            float s = 0.f;
#pragma unroll 8
            for (int r = 0; r < FS_ROWS; ++r) s += Z[r * FS_ZLD + cc];
            float* dst = ((tid < FS_HD) ? a.dEk : a.dEv) + e_row(a, b, k) * D + h * FS_HD + c;
            atomicAdd(dst, s);
        }
        // the next iteration's first __syncthreads orders these reads before A_sh / Z are rewritten:
        // A_sh is rewritten before that barrier, so close the iteration with one here.
        __syncthreads();
    }
    if (t < a.T) {
#pragma unroll
        for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<float4*>(a.dQ + qoff + i) = make_float4(dq[i], dq[i + 1], dq[i + 2], dq[i + 3]);
    }
    for (int j = 0; j < 4; ++j)
        if (wn + 32 * j < N)
            for (int i = 0; i < 8; ++i) part_out[(size_t)(wn + 32 * j) * FS_HD + wd + i] = dw[j][i];
}

// dW[n, h*64 + d] = sum over the CTAs of head h of part[cta][n][d]   (fixed order -> deterministic)
__global__ void k_flash_dw_reduce(const float* __restrict__ part, float* __restrict__ dW, int B, int H, int N,
                                  int ctas_per_bh) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int D = H * FS_HD;
    if (idx >= N * D) return;
    const int n = idx / D, col = idx % D, h = col / FS_HD, d = col % FS_HD;
    float s = 0.f;
    for (int b = 0; b < B; ++b)
        for (int c = 0; c < ctas_per_bh; ++c)
            s += part[((((size_t)b * H + h) * ctas_per_bh + c) * N + n) * FS_HD + d];
    dW[(size_t)n * D + col] = s;
}

static size_t fs_smem_fwd(int N) { return ((size_t)N * FS_HD + (size_t)round4(FS_ROWS * (N + 1)) + round4(N) + MBEMA_TILE_T) * 4; }
static size_t fs_smem_bwd(int N) { return fs_smem_fwd(N) + 3 * (size_t)FS_ROWS * FS_ZLD * 4; }

int flash_fwd_simt(const FlashArgs& a, cudaStream_t st) {
    const size_t smem = fs_smem_fwd(a.N);
    MBEMA_CUDA_TRY(cudaFuncSetAttribute(k_flash_fwd_simt, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(2 * a.nT, a.H, a.B);
    k_flash_fwd_simt<<<grid, FS_THREADS, smem, st>>>(a);
    return check_launch();
}

size_t flash_bwd_simt_ws(int64_t B, int64_t H, int64_t T, int64_t N) {
    const int64_t nT = (T + MBEMA_TILE_T - 1) / MBEMA_TILE_T;
    return (size_t)(B * H * 2 * nT) * (size_t)N * FS_HD * sizeof(float) + 256;
}

int flash_bwd_simt(FlashArgs a, float* dW, void* ws, cudaStream_t st) {
    const int D = a.H * FS_HD;
    a.dW_part = (float*)(((uintptr_t)ws + 255) / 256 * 256);
    MBEMA_CUDA_TRY(cudaMemsetAsync(a.dEk, 0, (size_t)a.e_rows * D * sizeof(float), st));
    MBEMA_CUDA_TRY(cudaMemsetAsync(a.dEv, 0, (size_t)a.e_rows * D * sizeof(float), st));
    const size_t smem = fs_smem_bwd(a.N);
    MBEMA_CUDA_TRY(cudaFuncSetAttribute(k_flash_bwd_simt, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(2 * a.nT, a.H, a.B);
    k_flash_bwd_simt<<<grid, FS_THREADS, smem, st>>>(a);
    int rc = check_launch();
    if (rc) return rc;
    const int total = a.N * D;
    k_flash_dw_reduce<<<(total + 255) / 256, 256, 0, st>>>(a.dW_part, dW, a.B, a.H, a.N, 2 * a.nT);
    return check_launch();
}

}  // namespace mbema
