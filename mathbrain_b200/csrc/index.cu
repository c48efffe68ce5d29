// Per-slot EMA state kernels: token sort/link, query-side chain scan, slot-state snapshots.
//
// The query-side state of token x_t depends only on the earlier occurrences of the same token, so the
// time axis of every sample is first regrouped by token: one CTA per sample sorts (token, t) pairs in
// shared memory (bitonic network), which turns every token's occurrences into one contiguous, time-ordered
// "chain".  A warp then walks a chain with the N channels spread over its lanes (coalesced 4*N-byte rows),
// carrying the fp32 state in registers:  c_t = (c_s + 1) * rho^(t - s).  The power is evaluated in double
// precision and rounded once: a token repeated at every step turns any bias of rho^1 into a state error
// amplified by 1 / (1 - rho).  No vocabulary-sized scratch is
// touched (the reference fills [B, V+1, N] floats per call, mathbrain/triton_ema_query.py:141-143).
#include <math.h>

#include <cuda_fp16.h>
#include <atomic>

#include "common.cuh"

namespace mbema {

static constexpr int SORT_THREADS = 1024;
static constexpr int NO_SEED = 0x7fffffff;

struct IndexWs {
    int32_t* s_tok;    // [B, T]  token of the j-th entry in (token, t) order
    int32_t* s_pos;    // [B, T]  its time step
    int32_t* ch_off;   // [B, T]  offset of the c-th chain head in the sorted order
    int32_t* seed;     // [B, T]  at a chain head: index of the first listed key equal to the token, or NO_SEED
    int32_t* n_chain;  // [B]
    int32_t* n_valid;  // [B]     number of keys >= 0
};

static size_t index_ws_bytes(int64_t B, int64_t T) {
    return align_up((size_t)(4 * B * T + 2 * B) * sizeof(int32_t), 256) + 256;
}

static IndexWs carve_index_ws(void* ws, int64_t B, int64_t T) {
    IndexWs w;
    uintptr_t p = (uintptr_t)ws;
    p = (p + 255) / 256 * 256;
    int32_t* base = (int32_t*)p;
    w.s_tok = base;
    w.s_pos = base + B * T;
    w.ch_off = base + 2 * B * T;
    w.seed = base + 3 * B * T;
    w.n_chain = base + 4 * B * T;
    w.n_valid = w.n_chain + B;
    return w;
}

// ----------------------------------------------------------------------------------------------
// one CTA per sample: sort (token, t), mark chain heads, compact them, attach listed keys
// dynamic smem: uint64 key[Tp] | int32 seed[Tp] | int32 scan[SORT_THREADS]
// ----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(SORT_THREADS)
k_sort_link(const int64_t* __restrict__ x, const int64_t* __restrict__ keys, IndexWs w, int T, int Tp, int K) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned long long* key = reinterpret_cast<unsigned long long*>(smem_raw);
    int* seed = reinterpret_cast<int*>(key + Tp);
    int* scan = seed + Tp;
    const int b = blockIdx.x;
    const int tid = threadIdx.x;

    for (int i = tid; i < Tp; i += SORT_THREADS) {
        unsigned long long kk = ~0ull;
        if (i < T) {
            unsigned long long tok = (unsigned long long)(x[(size_t)b * T + i]) & 0x7fffffffull;
            kk = (tok << 32) | (unsigned)i;
        }
        key[i] = kk;
        seed[i] = NO_SEED;
    }
    __syncthreads();
    for (int k = 2; k <= Tp; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = tid; i < Tp; i += SORT_THREADS) {
                int ixj = i ^ j;
                if (ixj > i) {
                    unsigned long long a = key[i], c = key[ixj];
                    bool up = ((i & k) == 0);
                    if ((a > c) == up) {
                        key[i] = c;
                        key[ixj] = a;
                    }
                }
            }
            __syncthreads();
        }
    }
    // chain heads: contiguous segment per thread, block-wide exclusive scan of the head counts
    const int per = (Tp + SORT_THREADS - 1) / SORT_THREADS;
    const int lo = tid * per;
    int cnt = 0;
    for (int i = lo; i < lo + per && i < T; ++i) {
        bool head = (i == 0) || ((key[i] >> 32) != (key[i - 1] >> 32));
        cnt += head ? 1 : 0;
    }
    scan[tid] = cnt;
    __syncthreads();
    for (int off = 1; off < SORT_THREADS; off <<= 1) {
        int v = (tid >= off) ? scan[tid - off] : 0;
        __syncthreads();
        scan[tid] += v;
        __syncthreads();
    }
    int c = scan[tid] - cnt;  // exclusive prefix
    int32_t* ch_off = w.ch_off + (size_t)b * T;
    for (int i = lo; i < lo + per && i < T; ++i) {
        bool head = (i == 0) || ((key[i] >> 32) != (key[i - 1] >> 32));
        if (head) ch_off[c++] = i;
    }
    if (tid == SORT_THREADS - 1) w.n_chain[b] = scan[tid];

    // listed keys -> chain heads (first listed entry wins)
    int nvalid = 0;
    if (keys != nullptr) {
        for (int i = tid; i < K; i += SORT_THREADS) {
            long long kv = keys[(size_t)b * K + i];
            if (kv < 0) continue;
            nvalid++;
            unsigned long long target = ((unsigned long long)kv & 0x7fffffffull) << 32;
            int l = 0, r = T;  // lower bound of target in key[0..T)
            while (l < r) {
                int m = (l + r) >> 1;
                if (key[m] < target) l = m + 1; else r = m;
            }
            if (l < T && (key[l] >> 32) == (target >> 32)) atomicMin(&seed[l], i);
        }
    }
    __syncthreads();
    scan[tid] = nvalid;
    __syncthreads();
    for (int off = SORT_THREADS / 2; off > 0; off >>= 1) {
        if (tid < off) scan[tid] += scan[tid + off];
        __syncthreads();
    }
    if (tid == 0) w.n_valid[b] = scan[0];
    for (int i = tid; i < T; i += SORT_THREADS) {
        w.s_tok[(size_t)b * T + i] = (int32_t)(key[i] >> 32);
        w.s_pos[(size_t)b * T + i] = (int32_t)(key[i] & 0xffffffffull);
        w.seed[(size_t)b * T + i] = seed[i];
    }
}

// ----------------------------------------------------------------------------------------------
// The workspace already holds the (token, t) order and the chain heads of the same x (left there by an earlier call):
// only the links from listed keys to chain heads are rebuilt, for a new key list.  One CTA per sample.
// ----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_relink(const int64_t* __restrict__ keys, IndexWs w, int T, int K) {
    __shared__ int cnt_sh;
    const int b = blockIdx.x, tid = threadIdx.x;
    int32_t* seed = w.seed + (size_t)b * T;
    const int32_t* s_tok = w.s_tok + (size_t)b * T;
    if (tid == 0) cnt_sh = 0;
    for (int i = tid; i < T; i += blockDim.x) seed[i] = NO_SEED;
    __syncthreads();
    int nvalid = 0;
    for (int i = tid; i < K; i += blockDim.x) {
        const long long kv = keys[(size_t)b * K + i];
        if (kv < 0) continue;
        nvalid++;
        const int key = (int)(kv & 0x7fffffff);
        int l = 0, r = T;            // lower bound: the first entry of the key's chain, if the token occurs
        while (l < r) {
            const int m = (l + r) >> 1;
            if (s_tok[m] < key) l = m + 1; else r = m;
        }
        if (l < T && s_tok[l] == key) atomicMin(&seed[l], i);      // first listed entry wins
    }
    atomicAdd(&cnt_sh, nvalid);
    __syncthreads();
    if (tid == 0) w.n_valid[b] = cnt_sh;
}

// ----------------------------------------------------------------------------------------------
// one warp per chain; lanes hold channels lane, lane+32, lane+64, lane+96
// ----------------------------------------------------------------------------------------------
static constexpr int CHAIN_WARPS = 8;
static constexpr int LONG_CHAIN = 64;      // occurrences from which a chain is scanned with warp shuffles instead of walked
static constexpr int COOP_BLOCKS = 2;      // CTAs per sample, at the end of the grid, that scan the long chains

// Long chains (the padding token, the most frequent tokens) are not walked but scanned: with U the carried value
// (state + 1 after the previous occurrence; the seed before the first), occurrence j reads v_j = A_j U_j and hands on
// U_{j+1} = A_j U_j + 1, A_j = keep_j rho^(t_j - t_{j-1}): an affine map per occurrence.  32 occurrences sit on the
// lanes and the maps are composed with warp shuffles (a segmented prefix product over time, five steps per block of
// 32); the N channels are split over the eight warps of the CTA, so a chain of L occurrences costs L/32 * N/8 short
// scans instead of L dependent steps.  Results go through shared memory so that a row's channels leave together.
__device__ void scan_long_chains(const IndexWs& w, const float* __restrict__ rhos, const float* __restrict__ c_init,
                                 const int32_t* __restrict__ doc_ids, float* __restrict__ out, int T, int N, int K,
                                 int extra_decay, int b, int q) {
    __shared__ int lst[8192 / LONG_CHAIN];
    __shared__ int n_long;
    __shared__ float tile[CHAIN_WARPS][32][17];
    __shared__ int tile_t[CHAIN_WARPS][32];
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const int nch = w.n_chain[b];
    const int32_t* ch_off = w.ch_off + (size_t)b * T;
    const int32_t* s_pos = w.s_pos + (size_t)b * T;
    if (tid == 0) n_long = 0;
    __syncthreads();
    for (int c = tid; c < nch; c += blockDim.x) {
        const int len = ((c + 1 < nch) ? ch_off[c + 1] : T) - ch_off[c];
        if (len >= LONG_CHAIN) lst[atomicAdd(&n_long, 1)] = c;
    }
    __syncthreads();
    const int nk = (N + CHAIN_WARPS - 1) / CHAIN_WARPS;          // channels of this warp: [wp * nk, wp * nk + nk)
    const int n_mine = wp * nk + lane;                           // lane k < nk keeps rho, its log and the carry of channel k
    const bool mine = lane < nk && n_mine < N;
    const float rho_k = mine ? rhos[n_mine] : 1.0f;
    const double l2r_k = mine ? log2((double)rho_k) : 0.0;
    int kmax = min(nk, N - wp * nk);
    if (kmax < 0) kmax = 0;
    for (int li = q; li < n_long; li += COOP_BLOCKS) {
        const int c = lst[li];
        const int j0 = ch_off[c];
        const int j1 = (c + 1 < nch) ? ch_off[c + 1] : T;
        const int sd = w.seed[(size_t)b * T + j0];
        float car = 0.0f;
        if (sd != NO_SEED && mine && c_init != nullptr) {
            car = c_init[((size_t)b * K + sd) * N + n_mine];
            if (extra_decay) car *= rho_k;
        }
        bool has = (sd != NO_SEED);
        int s_ref = 0;
        int last_doc = (doc_ids != nullptr) ? doc_ids[(size_t)b * T] : 0;
        for (int jb = j0; jb < j1; jb += 32) {
            const int cnt = min(32, j1 - jb);
            const bool live = lane < cnt;
            const int t_l = live ? s_pos[jb + lane] : 0;
            int t_prev = __shfl_up_sync(0xffffffffu, t_l, 1);
            if (lane == 0) t_prev = s_ref;
            bool keep = (lane == 0) ? has : true;
            if (doc_ids != nullptr) {
                const int d_l = live ? doc_ids[(size_t)b * T + t_l] : 0;
                int d_prev = __shfl_up_sync(0xffffffffu, d_l, 1);
                if (lane == 0) d_prev = last_doc;
                if (d_l != d_prev) keep = false;
                last_doc = __shfl_sync(0xffffffffu, d_l, cnt - 1);
            }
            const int di = t_l - t_prev;
            const double dt = (double)di;
            tile_t[wp][lane] = t_l;
            for (int k = 0; k < kmax; ++k) {
                const float rn = __shfl_sync(0xffffffffu, rho_k, k);
                const double l2 = __shfl_sync(0xffffffffu, l2r_k, k);
                // one step since the last occurrence: the decay is rho itself; longer gaps take the power in double
                float A = 0.f;
                if (live && keep) A = (di == 1) ? rn : (float)exp2(dt * l2);
                const float A_own = A;
                float Bv = live ? 1.0f : 0.0f;       // dead lanes carry the identity map: lane 31 ends with the last live result
                if (!live) A = 1.0f;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {    // inclusive composition with the maps of the earlier lanes
                    const float Ap = __shfl_up_sync(0xffffffffu, A, o), Bp = __shfl_up_sync(0xffffffffu, Bv, o);
                    if (lane >= o) { Bv = fmaf(A, Bp, Bv); A *= Ap; }
                }
                const float U_in = __shfl_sync(0xffffffffu, car, k);
                float Ae = __shfl_up_sync(0xffffffffu, A, 1), Be = __shfl_up_sync(0xffffffffu, Bv, 1);
                if (lane == 0) { Ae = 1.0f; Be = 0.0f; }
                tile[wp][lane][k] = A_own * fmaf(Ae, U_in, Be);                       // v_j = A_j U_j
                const float U_out = __shfl_sync(0xffffffffu, fmaf(A, U_in, Bv), 31);  // carried past the block
                if (lane == k) car = U_out;
            }
            __syncwarp();
            for (int idx = lane; idx < cnt * kmax; idx += 32) {
                const int r = idx / kmax, k = idx - r * kmax;
                out[((size_t)b * T + tile_t[wp][r]) * N + wp * nk + k] = tile[wp][r][k];
            }
            __syncwarp();
            s_ref = __shfl_sync(0xffffffffu, t_l, cnt - 1);
            has = true;
        }
    }
}

__global__ void __launch_bounds__(CHAIN_WARPS * 32)
k_chain_scan(IndexWs w, const float* __restrict__ rhos, const float* __restrict__ c_init,
             const int32_t* __restrict__ doc_ids, float* __restrict__ out, int T, int N, int K, int extra_decay) {
    const int b = blockIdx.y;
    if ((int)blockIdx.x >= (int)gridDim.x - COOP_BLOCKS) {
        scan_long_chains(w, rhos, c_init, doc_ids, out, T, N, K, extra_decay, b, (int)blockIdx.x - ((int)gridDim.x - COOP_BLOCKS));
        return;
    }
    const int c = blockIdx.x * CHAIN_WARPS + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int nch = w.n_chain[b];
    if (c >= nch) return;
    const int32_t* ch_off = w.ch_off + (size_t)b * T;
    const int32_t* s_pos = w.s_pos + (size_t)b * T;
    const int j0 = ch_off[c];
    const int j1 = (c + 1 < nch) ? ch_off[c + 1] : T;
    const int sd = w.seed[(size_t)b * T + j0];

    double l2r[4];
    float u[4], rho[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int n = lane + 32 * i;
        float r = (n < N) ? rhos[n] : 1.0f;
        rho[i] = r;
        l2r[i] = (32 * i < N) ? log2((double)r) : 0.0;
        u[i] = 0.0f;
        if (sd != NO_SEED && n < N && c_init != nullptr) {
            u[i] = c_init[((size_t)b * K + sd) * N + n];
            if (extra_decay) u[i] *= r;
        }
    }
    bool has = (sd != NO_SEED);
    int s_ref = 0;
    int last_doc = (doc_ids != nullptr) ? doc_ids[(size_t)b * T] : 0;
    if (j1 - j0 >= LONG_CHAIN) return;      // scanned by the cooperative blocks at the end of the grid
    // The chain is walked 32 occurrences at a time: every lane fetches one position (and document id), the steps then
    // take them from registers with shuffles, so a long chain pays the load latency once per 32 steps, not per step.
    for (int jb = j0; jb < j1; jb += 32) {
        const int jj = jb + lane;
        const int t_l = (jj < j1) ? s_pos[jj] : 0;
        const int d_l = (doc_ids != nullptr && jj < j1) ? doc_ids[(size_t)b * T + t_l] : 0;
        const int cnt = min(32, j1 - jb);
        for (int q = 0; q < cnt; ++q) {
            const int t = __shfl_sync(0xffffffffu, t_l, q);
            bool keep = has;
            if (doc_ids != nullptr) {
                const int d = __shfl_sync(0xffffffffu, d_l, q);
                if (has && d != last_doc) keep = false;
                last_doc = d;
            }
            const int di = t - s_ref;
            const double dt = (double)di;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (32 * i < N) {   // channel groups beyond N do nothing
                    int n = lane + 32 * i;
                    // one step since the last occurrence (runs of a repeated token, e.g. the padding): the decay is
                    // rho itself; longer gaps take the power in double precision (its error is amplified by
                    // 1 / (1 - rho))
                    const float pw = (di == 1) ? rho[i] : (float)exp2(dt * l2r[i]);
                    float cval = keep ? u[i] * pw : 0.0f;
                    if (n < N) out[((size_t)b * T + t) * N + n] = cval;
                    u[i] = cval + 1.0f;
                }
            }
            s_ref = t;
            has = true;
        }
    }
}

// ----------------------------------------------------------------------------------------------
// one warp per listed slot: state at the start of every time tile
// ----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(CHAIN_WARPS * 32)
k_tile_states(IndexWs w, const int64_t* __restrict__ unique, const float* __restrict__ rhos,
              const float* __restrict__ c_base, float* __restrict__ tile_state, int T, int N, int K, int nT,
              int extra_decay) {
    extern __shared__ float pw_sh[];            // [nT][N]: rho_n^(tile * 128), evaluated in double precision
    for (int i = threadIdx.x; i < nT * N; i += blockDim.x)
        pw_sh[i] = (float)exp2((double)((i / N) * MBEMA_TILE_T) * log2((double)rhos[i % N]));
    __syncthreads();
    const int b = blockIdx.y;
    const int k = blockIdx.x * CHAIN_WARPS + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (k >= K) return;
    const long long kv = unique[(size_t)b * K + k];
    const int32_t* s_tok = w.s_tok + (size_t)b * T;
    const int32_t* s_pos = w.s_pos + (size_t)b * T;
    float* out = tile_state + ((size_t)b * nT * K + k) * N;  // + tile * K * N
    // the same snapshots in 16 bits follow the fp32 block (operand format of the tensor-core attention kernels:
    // fp16 of state / 64)
    __nv_bfloat16* out16 = reinterpret_cast<__nv_bfloat16*>(tile_state + (size_t)gridDim.y * nT * K * N) +
                           ((size_t)b * nT * K + k) * N;
    if (kv < 0) {
        for (int i = 0; i < nT; ++i)
            for (int n = lane; n < N; n += 32) {
                out[(size_t)i * K * N + n] = 0.0f;
                out16[(size_t)i * K * N + n] = __float2bfloat16(0.0f);   // +0 in fp16 as well
            }
        return;
    }
    const int key = (int)(kv & 0x7fffffff);
    int l = 0, r = T;
    while (l < r) {
        int m = (l + r) >> 1;
        if (s_tok[m] < key) l = m + 1; else r = m;
    }
    int j = l;
    double l2r[4];
    float u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int n = lane + 32 * i;
        float rr = (n < N) ? rhos[n] : 1.0f;
        l2r[i] = (32 * i < N) ? log2((double)rr) : 0.0;
        u[i] = 0.0f;
        if (c_base != nullptr && n < N) {
            u[i] = c_base[((size_t)b * K + k) * N + n];
            if (extra_decay) u[i] *= rr;
        }
    }
    int s_ref = 0;
    // occurrences are read 32 at a time (one per lane) and handed out with shuffles: `blk` is the first index of the
    // block in registers; positions of other tokens or beyond T read as "no more occurrences"
    int blk = -64, pos_l = 0x7fffffff;
    auto occurrence = [&](int jx) -> int {       // step of the jx-th sorted entry if it is an occurrence of `key`, else INT_MAX
        if (jx - blk >= 32) {
            blk = jx;
            const int jj = jx + lane;
            pos_l = (jj < T && s_tok[jj] == key) ? s_pos[jj] : 0x7fffffff;
        }
        return __shfl_sync(0xffffffffu, pos_l, jx - blk);
    };
    for (int tile = 0; tile < nT; ++tile) {
        const int t0 = tile * MBEMA_TILE_T;
        for (int s = occurrence(j); s < t0; s = occurrence(j)) {
            const double dt = (double)(s - s_ref);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (32 * i < N) u[i] = u[i] * (float)exp2(dt * l2r[i]) + 1.0f;
            s_ref = s;
            ++j;
        }
        const double dt = (double)(t0 - s_ref);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int n = lane + 32 * i;
            if (32 * i < N && n < N) {
                // no occurrence yet: the power rho^t0 is the same for every slot of the CTA (table in shared memory)
                const float pw = (s_ref == 0) ? pw_sh[tile * N + n] : (float)exp2(dt * l2r[i]);
                const float v = u[i] * pw;
                out[(size_t)tile * K * N + n] = v;
                // operand format of the tensor-core attention kernels: fp16 of state / 64, saturated
                reinterpret_cast<__half*>(out16)[(size_t)tile * K * N + n] = __float2half_rn(fminf(v * (1.0f / 64.0f), 65504.0f));
            }
        }
    }
}

// order[r] = sample with the r-th largest number of valid slots (ties by index): heavy samples are scheduled first
__global__ void k_slot_order(const int32_t* __restrict__ n_valid, int32_t* __restrict__ kcount, int B) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const int mine = n_valid[b];
    kcount[b] = mine;
    int rank = 0;
    if (B <= 4096) {
        for (int j = 0; j < B; ++j) {
            const int o = n_valid[j];
            rank += (o > mine || (o == mine && j < b)) ? 1 : 0;
        }
    } else {
        rank = b;
    }
    kcount[B + rank] = b;
}

static int launch_sort_link(const int64_t* x, const int64_t* keys, IndexWs w, int64_t B, int64_t T, int64_t K,
                            cudaStream_t st) {
    int Tp = 2;
    while (Tp < T) Tp <<= 1;
    size_t smem = (size_t)Tp * 12 + SORT_THREADS * 4;
    // per-device attribute; setting it on every call keeps the library free of per-device bookkeeping
    MBEMA_CUDA_TRY(cudaFuncSetAttribute(k_sort_link, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        8192 * 12 + SORT_THREADS * 4));
    k_sort_link<<<(unsigned)B, SORT_THREADS, smem, st>>>(x, keys, w, (int)T, Tp, (int)K);
    return check_launch();
}

}  // namespace mbema

using namespace mbema;

extern "C" size_t mbema_query_scan_workspace_bytes(int64_t B, int64_t T) { return index_ws_bytes(B, T); }
extern "C" size_t mbema_tile_states_workspace_bytes(int64_t B, int64_t T) { return index_ws_bytes(B, T); }

static int check_index_args(int64_t B, int64_t T, int64_t N, int64_t K) {
    if (B < 0 || T < 1 || N < 1 || K < 0) return MBEMA_ERR_SHAPE;
    if (T > 8192 || N > 128 || B > 65535) return MBEMA_ERR_UNSUPPORTED;
    return MBEMA_OK;
}

extern "C" int mbema_query_scan(const int64_t* x, const float* rhos, const float* c_init, const int64_t* c_init_keys,
                                const int32_t* doc_ids, float* C_seq, int64_t B, int64_t T, int64_t N, int64_t K,
                                int flags, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_index_args(B, T, N, K);
    if (rc) return rc;
    if (B == 0) return MBEMA_OK;
    if (!x || !rhos || !C_seq || !workspace) return MBEMA_ERR_NULL;
    if ((c_init == nullptr) != (c_init_keys == nullptr)) return MBEMA_ERR_NULL;
    if (workspace_bytes < index_ws_bytes(B, T)) return MBEMA_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    IndexWs w = carve_index_ws(workspace, B, T);
    rc = launch_sort_link(x, c_init_keys, w, B, T, c_init_keys ? K : 0, st);
    if (rc) return rc;
    dim3 grid((unsigned)((T + CHAIN_WARPS - 1) / CHAIN_WARPS + COOP_BLOCKS), (unsigned)B);
    k_chain_scan<<<grid, CHAIN_WARPS * 32, 0, st>>>(w, rhos, c_init, doc_ids, C_seq, (int)T, (int)N, (int)K,
                                                    (flags & MBEMA_FLAG_CBASE_EXTRA_DECAY) ? 1 : 0);
    return check_launch();
}

extern "C" int mbema_tile_states(const int64_t* x, const int64_t* unique, const float* rhos, const float* c_base,
                                 float* tile_state, float* tok_state, int32_t* kcount, int64_t B, int64_t T,
                                 int64_t N, int64_t K, int flags, void* workspace, size_t workspace_bytes,
                                 void* stream) {
    int rc = check_index_args(B, T, N, K);
    if (rc) return rc;
    if (B == 0) return MBEMA_OK;
    if (K < 1) return MBEMA_ERR_SHAPE;
    if (!x || !unique || !rhos || !tile_state || !tok_state || !kcount || !workspace) return MBEMA_ERR_NULL;
    if (workspace_bytes < index_ws_bytes(B, T)) return MBEMA_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    IndexWs w = carve_index_ws(workspace, B, T);
    const int extra = (flags & MBEMA_FLAG_CBASE_EXTRA_DECAY) ? 1 : 0;
    if (flags & MBEMA_FLAG_INDEX_READY) {     // the sort of this x is in the workspace already: new key links only
        k_relink<<<(unsigned)B, 256, 0, st>>>(unique, w, (int)T, (int)K);
        rc = check_launch();
    } else {
        rc = launch_sort_link(x, unique, w, B, T, K, st);
    }
    if (rc) return rc;
    dim3 g1((unsigned)((T + CHAIN_WARPS - 1) / CHAIN_WARPS + COOP_BLOCKS), (unsigned)B);
    // a chain without a listed key keeps zero state in tok_state only if it is unlisted: such tokens own no slot,
    // so their rows are never read by the attention kernels; they are still written (query-scan semantics).
    k_chain_scan<<<g1, CHAIN_WARPS * 32, 0, st>>>(w, rhos, c_base, nullptr, tok_state, (int)T, (int)N, (int)K, extra);
    rc = check_launch();
    if (rc) return rc;
    const int nT = (int)((T + MBEMA_TILE_T - 1) / MBEMA_TILE_T);
    dim3 g2((unsigned)((K + CHAIN_WARPS - 1) / CHAIN_WARPS), (unsigned)B);
    k_tile_states<<<g2, CHAIN_WARPS * 32, (size_t)nT * N * sizeof(float), st>>>(w, unique, rhos, c_base, tile_state, (int)T, (int)N, (int)K, nT, extra);
    rc = check_launch();
    if (rc) return rc;
    k_slot_order<<<(unsigned)((B + 127) / 128), 128, 0, st>>>(w.n_valid, kcount, (int)B);
    return check_launch();
}

// ------------------------------------------------------------------------------------------------
// Query scan without any allocation on the caller's side: the index scratch lives in a fixed device array.
// ------------------------------------------------------------------------------------------------
#define MBEMA_STATIC_SCAN_MAX_TOKENS 32768   /* B * T */
#define MBEMA_STATIC_SCAN_MAX_BATCH 1024

namespace mbema {
// Scratch of the allocation-free scan: 4 int32 per token + 2 per sample, plus alignment slack (~0.5 MB).  Every GPU
// that loads the library carries this array until the process exits.
static __device__ __align__(256) int32_t g_static_scan_scratch[4 * MBEMA_STATIC_SCAN_MAX_TOKENS + 2 * MBEMA_STATIC_SCAN_MAX_BATCH + 128];
static constexpr int MAX_DEVICES = 64;
// device address of the array, per device, filled on first use; atomic because two host threads may make their first
// call on the same device at the same time (both look the address up and store the same value)
static std::atomic<void*> g_static_scan_addr[MAX_DEVICES];
}  // namespace mbema

extern "C" int mbema_query_scan_static(const int64_t* x, const float* rhos, const float* c_init,
                                       const int64_t* c_init_keys, const int32_t* doc_ids, float* C_seq, int64_t B,
                                       int64_t T, int64_t N, int64_t K, int flags, void* stream) {
    int rc = check_index_args(B, T, N, K);
    if (rc) return rc;
    if (B == 0) return MBEMA_OK;
    if (B * T > MBEMA_STATIC_SCAN_MAX_TOKENS || B > MBEMA_STATIC_SCAN_MAX_BATCH) return MBEMA_ERR_STATIC_LIMIT;
    if (!x || !rhos || !C_seq) return MBEMA_ERR_NULL;
    if ((c_init == nullptr) != (c_init_keys == nullptr)) return MBEMA_ERR_NULL;
    int dev = 0;
    MBEMA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return MBEMA_ERR_UNSUPPORTED;
    void* scratch = g_static_scan_addr[dev].load(std::memory_order_acquire);
    if (scratch == nullptr) {
        // In host code the array's name is only a handle; the kernels need its address on the current device.
        MBEMA_CUDA_TRY(cudaGetSymbolAddress(&scratch, g_static_scan_scratch));
        g_static_scan_addr[dev].store(scratch, std::memory_order_release);
    }
    cudaStream_t st = (cudaStream_t)stream;
    IndexWs w = carve_index_ws(scratch, B, T);
    rc = launch_sort_link(x, c_init_keys, w, B, T, c_init_keys ? K : 0, st);
    if (rc) return rc;
    dim3 grid((unsigned)((T + CHAIN_WARPS - 1) / CHAIN_WARPS + COOP_BLOCKS), (unsigned)B);
    k_chain_scan<<<grid, CHAIN_WARPS * 32, 0, st>>>(w, rhos, c_init, doc_ids, C_seq, (int)T, (int)N, (int)K,
                                                    (flags & MBEMA_FLAG_CBASE_EXTRA_DECAY) ? 1 : 0);
    return check_launch();
}
