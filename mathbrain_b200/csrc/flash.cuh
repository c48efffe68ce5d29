// Argument block and internal entry points shared by the attention kernels.
#pragma once
#include "common.cuh"

namespace mbema {

struct FlashArgs {
    const void* Q; int q_dt;
    const long long* x;
    const void* Ek; const void* Ev; int e_dt;
    const float* W; const float* rhos;
    const long long* unique;
    const float* tile_state; const float* tok_state;
    const int* kcount; const int* seq_lens;
    const int* order;   // [B] sample processed by blockIdx.z (heaviest first), or null
    const int* erow;    // [B, K] row of E_k / E_v / dE_k / dE_v that slot (b, k) uses, or null: row b * K + k
    long long e_rows;   // number of rows of E_k / E_v (B * K without erow)
    float* O; float* LSE;
    // backward only
    const void* dO; int do_dt;
    float* dQ; float* dEk; float* dEv; float* dW_part;
    int B, H, T, N, K, nT;
    float v_total;
    int silu, listed_only;
    int test_withhold;      // test hook: see MBEMA_FLAG_TEST_WITHHOLD_ARRIVE
};

// row of the slot-embedding tables (and of their gradients) that slot (b, k) reads
__device__ __forceinline__ size_t e_row(const FlashArgs& a, int b, int k) {
    return a.erow ? (size_t)a.erow[(size_t)b * a.K + k] : (size_t)b * a.K + k;
}

int flash_fwd_simt(const FlashArgs& a, cudaStream_t st);
size_t flash_bwd_simt_ws(int64_t B, int64_t H, int64_t T, int64_t N);
int flash_bwd_simt(FlashArgs a, float* dW, void* ws, cudaStream_t st);

// tensor-core (tcgen05) path
bool flash_tc_supported(int H, int N, int K);
size_t flash_fwd_tc_ws();
int flash_fwd_tc(const FlashArgs& a, void* ws, cudaStream_t st);
bool flash_bwd_tc_supported(int H, int N, int K);
size_t flash_bwd_tc_ws(int64_t B, int64_t H, int64_t T, int64_t N);
int flash_bwd_tc(FlashArgs a, float* dW, void* ws, cudaStream_t st);

}  // namespace mbema
