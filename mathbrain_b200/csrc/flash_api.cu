// C entry points of the flash-EMA attention: argument checks and dispatch on the compute mode.
#include "flash.cuh"

using namespace mbema;

static bool dt_ok(int dt) { return dt == MBEMA_F32 || dt == MBEMA_BF16; }

static int flash_check(int64_t B, int64_t H, int64_t T, int64_t hd, int64_t N, int64_t K, int mode) {
    if (B < 0 || H < 1 || T < 1 || N < 1 || K < 1) return MBEMA_ERR_SHAPE;
    if (hd != 64 || N > 128 || T > 8192 || B > 65535 || H > 65535) return MBEMA_ERR_UNSUPPORTED;
    if (mode != MBEMA_MODE_FP32 && mode != MBEMA_MODE_TC_BF16) return MBEMA_ERR_UNSUPPORTED;
    if (mode == MBEMA_MODE_TC_BF16 && !flash_tc_supported((int)H, (int)N, (int)K)) return MBEMA_ERR_UNSUPPORTED;
    return MBEMA_OK;
}

static FlashArgs pack(const void* Q, int q_dtype, const int64_t* x, const void* E_k, const void* E_v, int e_dtype,
                      const float* W_pe, const float* rhos, const int64_t* unique, const float* tile_state,
                      const float* tok_state, const int32_t* kcount, const int32_t* seq_lens, int64_t B, int64_t H,
                      int64_t T, int64_t N, int64_t K, int64_t V_total, int flags) {
    FlashArgs a{};
    a.Q = Q; a.q_dt = q_dtype; a.x = (const long long*)x; a.Ek = E_k; a.Ev = E_v; a.e_dt = e_dtype;
    a.W = W_pe; a.rhos = rhos; a.unique = (const long long*)unique; a.tile_state = tile_state;
    a.tok_state = tok_state; a.kcount = kcount; a.seq_lens = seq_lens;
    a.order = kcount + B;
    a.B = (int)B; a.H = (int)H; a.T = (int)T; a.N = (int)N; a.K = (int)K;
    a.nT = (int)((T + MBEMA_TILE_T - 1) / MBEMA_TILE_T);
    a.v_total = (float)V_total;
    a.silu = (flags & MBEMA_FLAG_SILU) ? 1 : 0;
    a.listed_only = (flags & MBEMA_FLAG_LISTED_ONLY) ? 1 : 0;
    a.test_withhold = (flags & MBEMA_FLAG_TEST_WITHHOLD_ARRIVE) ? 1 : 0;
    a.erow = nullptr;
    a.e_rows = (long long)B * K;
    return a;
}

extern "C" int mbema_flash_tc_supported(int64_t H, int64_t N, int64_t K) {
    if (H < 1 || N < 1 || K < 1 || H > 65535 || K > (1 << 20)) return 0;
    return flash_tc_supported((int)H, (int)N, (int)K) ? 1 : 0;
}

extern "C" size_t mbema_flash_fwd_workspace_bytes(int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int) {
    return 256;
}

static int flash_fwd_impl(const void* Q, int q_dtype, const int64_t* x, const void* E_k, const void* E_v,
                          int e_dtype, const int32_t* e_row_index, int64_t e_rows, const float* W_pe, const float* rhos,
                          const int64_t* unique, const float* tile_state, const float* tok_state, const int32_t* kcount,
                          const int32_t* seq_lens, float* O, float* LSE, int64_t B, int64_t H, int64_t T,
                          int64_t hd, int64_t N, int64_t K, int64_t V_total, int flags, int mode,
                          void* workspace, size_t workspace_bytes, void* stream) {
    int rc = flash_check(B, H, T, hd, N, K, mode);
    if (rc) return rc;
    if (e_row_index && e_rows < 1) return MBEMA_ERR_SHAPE;
    if (B == 0) return MBEMA_OK;
    if (!Q || !x || !E_k || !E_v || !W_pe || !rhos || !unique || !tile_state || !tok_state || !kcount || !O || !LSE)
        return MBEMA_ERR_NULL;
    if (!dt_ok(q_dtype) || !dt_ok(e_dtype)) return MBEMA_ERR_DTYPE;
    if (((uintptr_t)Q | (uintptr_t)E_k | (uintptr_t)E_v | (uintptr_t)O | (uintptr_t)W_pe | (uintptr_t)tile_state |
         (uintptr_t)tok_state) & 15)      // all of these are read with 16-byte vector or cp.async accesses
        return MBEMA_ERR_ALIGN;
    FlashArgs a = pack(Q, q_dtype, x, E_k, E_v, e_dtype, W_pe, rhos, unique, tile_state, tok_state, kcount, seq_lens,
                       B, H, T, N, K, V_total, flags);
    a.O = O; a.LSE = LSE;
    if (e_row_index) { a.erow = e_row_index; a.e_rows = e_rows; }
    if (mode == MBEMA_MODE_TC_BF16) {
        if (!workspace) return MBEMA_ERR_NULL;
        if (workspace_bytes < flash_fwd_tc_ws()) return MBEMA_ERR_WORKSPACE;
        return flash_fwd_tc(a, workspace, (cudaStream_t)stream);
    }
    return flash_fwd_simt(a, (cudaStream_t)stream);
}

extern "C" int mbema_flash_fwd(const void* Q, int q_dtype, const int64_t* x, const void* E_k, const void* E_v,
                               int e_dtype, const float* W_pe, const float* rhos, const int64_t* unique,
                               const float* tile_state, const float* tok_state, const int32_t* kcount,
                               const int32_t* seq_lens, float* O, float* LSE, int64_t B, int64_t H, int64_t T,
                               int64_t hd, int64_t N, int64_t K, int64_t V_total, int flags, int mode,
                               void* workspace, size_t workspace_bytes, void* stream) {
    return flash_fwd_impl(Q, q_dtype, x, E_k, E_v, e_dtype, nullptr, 0, W_pe, rhos, unique, tile_state, tok_state, kcount,
                          seq_lens, O, LSE, B, H, T, hd, N, K, V_total, flags, mode, workspace, workspace_bytes, stream);
}

extern "C" int mbema_flash_fwd_rows(const void* Q, int q_dtype, const int64_t* x, const void* E_k, const void* E_v,
                                    int e_dtype, const int32_t* e_row_index, int64_t e_rows, const float* W_pe,
                                    const float* rhos, const int64_t* unique, const float* tile_state,
                                    const float* tok_state, const int32_t* kcount, const int32_t* seq_lens, float* O,
                                    float* LSE, int64_t B, int64_t H, int64_t T, int64_t hd, int64_t N, int64_t K,
                                    int64_t V_total, int flags, int mode, void* workspace, size_t workspace_bytes,
                                    void* stream) {
    if (!e_row_index) return MBEMA_ERR_NULL;
    return flash_fwd_impl(Q, q_dtype, x, E_k, E_v, e_dtype, e_row_index, e_rows, W_pe, rhos, unique, tile_state, tok_state,
                          kcount, seq_lens, O, LSE, B, H, T, hd, N, K, V_total, flags, mode, workspace, workspace_bytes,
                          stream);
}

extern "C" size_t mbema_flash_bwd_workspace_bytes(int64_t B, int64_t H, int64_t T, int64_t hd, int64_t N, int64_t K,
                                                  int mode) {
    (void)hd;
    // in tensor-core mode the first 512 bytes hold the kernel status word, whichever kernel ends up running
    size_t need = flash_bwd_simt_ws(B, H, T, N) + (mode == MBEMA_MODE_TC_BF16 ? 512 : 0);
    if (mode == MBEMA_MODE_TC_BF16 && flash_bwd_tc_supported((int)H, (int)N, (int)K)) {
        const size_t tc = flash_bwd_tc_ws(B, H, T, N);
        if (tc > need) need = tc;
    }
    return need;
}

static int flash_bwd_impl(const void* Q, int q_dtype, const int64_t* x, const void* E_k, const void* E_v,
                          int e_dtype, const int32_t* e_row_index, int64_t e_rows, const float* W_pe, const float* rhos,
                          const int64_t* unique, const float* tile_state, const float* tok_state, const int32_t* kcount,
                          const int32_t* seq_lens, const float* O, const float* LSE, const void* dO,
                          int do_dtype, float* dQ, float* dE_k, float* dE_v, float* dW_pe, int64_t B, int64_t H,
                          int64_t T, int64_t hd, int64_t N, int64_t K, int64_t V_total, int flags, int mode,
                          void* workspace, size_t workspace_bytes, void* stream) {
    int rc = flash_check(B, H, T, hd, N, K, mode);
    if (rc) return rc;
    if (e_row_index && e_rows < 1) return MBEMA_ERR_SHAPE;
    if (!dW_pe) return MBEMA_ERR_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    if (B == 0) {
        MBEMA_CUDA_TRY(cudaMemsetAsync(dW_pe, 0, (size_t)N * H * hd * sizeof(float), st));
        return MBEMA_OK;
    }
    if (!Q || !x || !E_k || !E_v || !W_pe || !rhos || !unique || !tile_state || !tok_state || !kcount || !O || !LSE ||
        !dO || !dQ || !dE_k || !dE_v || !workspace)
        return MBEMA_ERR_NULL;
    if (!dt_ok(q_dtype) || !dt_ok(e_dtype) || !dt_ok(do_dtype)) return MBEMA_ERR_DTYPE;
    if (((uintptr_t)Q | (uintptr_t)E_k | (uintptr_t)E_v | (uintptr_t)O | (uintptr_t)dO | (uintptr_t)dQ | (uintptr_t)W_pe |
         (uintptr_t)tile_state | (uintptr_t)tok_state | (uintptr_t)dE_k | (uintptr_t)dE_v | (uintptr_t)dW_pe) & 15)
        return MBEMA_ERR_ALIGN;
    if (workspace_bytes < mbema_flash_bwd_workspace_bytes(B, H, T, hd, N, K, mode)) return MBEMA_ERR_WORKSPACE;
    FlashArgs a = pack(Q, q_dtype, x, E_k, E_v, e_dtype, W_pe, rhos, unique, tile_state, tok_state, kcount, seq_lens,
                       B, H, T, N, K, V_total, flags);
    a.O = const_cast<float*>(O); a.LSE = const_cast<float*>(LSE);
    a.dO = dO; a.do_dt = do_dtype; a.dQ = dQ; a.dEk = dE_k; a.dEv = dE_v;
    if (e_row_index) { a.erow = e_row_index; a.e_rows = e_rows; }
    // tensor-core backward where the shape fits its shared-memory budget (N == 64); otherwise the fp32 kernels
    if (mode == MBEMA_MODE_TC_BF16) {
        if (!(flags & MBEMA_FLAG_FP32_BACKWARD) && flash_bwd_tc_supported((int)H, (int)N, (int)K))
            return flash_bwd_tc(a, dW_pe, workspace, st);
        // (the first 512 bytes stay reserved for the status word of the tensor-core kernels; the fp32 kernels have no
        // bounded waits and leave it alone)
        return flash_bwd_simt(a, dW_pe, static_cast<unsigned char*>(workspace) + 512, st);
    }
    return flash_bwd_simt(a, dW_pe, workspace, st);
}

extern "C" int mbema_flash_bwd(const void* Q, int q_dtype, const int64_t* x, const void* E_k, const void* E_v,
                               int e_dtype, const float* W_pe, const float* rhos, const int64_t* unique,
                               const float* tile_state, const float* tok_state, const int32_t* kcount,
                               const int32_t* seq_lens, const float* O, const float* LSE, const void* dO,
                               int do_dtype, float* dQ, float* dE_k, float* dE_v, float* dW_pe, int64_t B, int64_t H,
                               int64_t T, int64_t hd, int64_t N, int64_t K, int64_t V_total, int flags, int mode,
                               void* workspace, size_t workspace_bytes, void* stream) {
    return flash_bwd_impl(Q, q_dtype, x, E_k, E_v, e_dtype, nullptr, 0, W_pe, rhos, unique, tile_state, tok_state, kcount,
                          seq_lens, O, LSE, dO, do_dtype, dQ, dE_k, dE_v, dW_pe, B, H, T, hd, N, K, V_total, flags, mode,
                          workspace, workspace_bytes, stream);
}

extern "C" int mbema_flash_bwd_rows(const void* Q, int q_dtype, const int64_t* x, const void* E_k, const void* E_v,
                                    int e_dtype, const int32_t* e_row_index, int64_t e_rows, const float* W_pe,
                                    const float* rhos, const int64_t* unique, const float* tile_state,
                                    const float* tok_state, const int32_t* kcount, const int32_t* seq_lens,
                                    const float* O, const float* LSE, const void* dO, int do_dtype, float* dQ,
                                    float* dE_k, float* dE_v, float* dW_pe, int64_t B, int64_t H, int64_t T, int64_t hd,
                                    int64_t N, int64_t K, int64_t V_total, int flags, int mode, void* workspace,
                                    size_t workspace_bytes, void* stream) {
    if (!e_row_index) return MBEMA_ERR_NULL;
    return flash_bwd_impl(Q, q_dtype, x, E_k, E_v, e_dtype, e_row_index, e_rows, W_pe, rhos, unique, tile_state, tok_state,
                          kcount, seq_lens, O, LSE, dO, do_dtype, dQ, dE_k, dE_v, dW_pe, B, H, T, hd, N, K, V_total, flags,
                          mode, workspace, workspace_bytes, stream);
}
