// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the attention kernels use:
// mbarrier, tcgen05 (TMEM allocation, UMMA issue/commit, TMEM loads), proxy fences.
// Every wait is bounded: after MBEMA_SPIN_LIMIT polls it gives up, raises the CTA's abort flag and returns,
// so a protocol error ends the kernel with an error status instead of hanging the GPU.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mbema {
namespace ptx {

static constexpr unsigned MBEMA_SPIN_LIMIT = 1u << 21;   // polls before a wait gives up (each poll may block briefly)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}

// One poll: the hardware may park the thread for a short, implementation-defined time before it answers.
// (No suspend-time hint: with a long hint the woken threads resumed late and the kernels ran slower.)
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait. `abort_flag` lives in shared memory; once set (by any thread) every later wait returns at once.
// A wait that expires stores 1 | (tag << 8) there, so the status word the kernel reports names the wait that gave up.
// SLEEP_NS > 0: the thread sleeps that long between polls.  A polling warp executes instructions, and those take issue
// slots from the warps that have work, so warps that wait far ahead of their consumer should poll rarely.
// `limit_ptr` (shared memory, optional): poll limit set by a test hook; it is read only after the first poll has failed, so
// the common case costs one try_wait and a branch and keeps no extra value in a register (a run-time limit held in a
// register across the kernel made the backward 14 % slower).
template <unsigned SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int tag = 0,
                                          const volatile unsigned* limit_ptr = nullptr) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned limit = limit_ptr ? *limit_ptr : MBEMA_SPIN_LIMIT;
    for (unsigned it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
        if ((it & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1 | (tag << 8);
    return false;
}

// barrier `id` (1..15) among `nthreads` threads of the CTA (a multiple of 32: whole warps)
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// make generic-proxy shared-memory writes visible to the async proxy (UMMA operand reads)
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// TMEM allocation: executed by one full warp; the base address is written to *slot (shared memory)
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                         // leading byte offset (unused for swizzled K-major), bits [16,30)
    d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset, bits [32,46)
    d |= (uint64_t)1 << 46;                         // descriptor version (Blackwell), bits [46,48)
    d |= (uint64_t)2 << 61;                         // layout type SWIZZLE_128B, bits [61,64)
    return d;
}

// Shared-memory matrix descriptor: MN-major operand, 128-byte swizzle.  The tile is stored as blocks of
// [8 K-rows][64 MN-elements] (1024 B, 128-byte rows swizzled like the K-major case); `lbo_bytes` is the distance
// between blocks that are adjacent in the MN direction, `sbo_bytes` between blocks adjacent in the K direction.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulation.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_bf16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// mbarrier arrive once all UMMAs previously issued by this thread have completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives row (lane base + i)
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// The two helpers below keep the compiler free to schedule unrelated arithmetic across a TMEM load and its wait: they
// carry no memory clobber, and the wait names the loaded registers as in/out operands, which orders every use of the
// loaded values after the wait (volatile asm statements keep their own order).
__device__ __forceinline__ void tmem_ld16_nb(uint32_t taddr, float (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]),
          "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld16(float (&v)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+f"(v[0]), "+f"(v[1]), "+f"(v[2]), "+f"(v[3]), "+f"(v[4]), "+f"(v[5]), "+f"(v[6]), "+f"(v[7]), "+f"(v[8]),
                   "+f"(v[9]), "+f"(v[10]), "+f"(v[11]), "+f"(v[12]), "+f"(v[13]), "+f"(v[14]), "+f"(v[15]));
}

__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const float* v) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// one 16-byte shared-memory store (kept as a single instruction: four separate 4-byte stores from a warp whose
// lanes are 128 bytes apart would all hit the same banks)
__device__ __forceinline__ void st_shared_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(smem_u32(p)), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed fp32 pairs (sm_100 f32x2 arithmetic): one FMA-pipe instruction per two elements.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }
// tanh of both bf16 halves (one MUFU operation for the pair)
__device__ __forceinline__ uint32_t tanh_bf16x2(uint32_t a) {
    uint32_t d;
    asm("tanh.approx.bf16x2 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
// ---- fp16 pairs: the state tiles of the N = 64 kernels are fp16 (11 significant bits against bf16's 8), stored
// scaled by STATE_F16_SCALE so that every reachable state stays below the fp16 maximum
static constexpr float STATE_F16_SCALE = 1.0f / 64.0f;     // state / 64 <= 65504  <=>  state <= 4.19e6
static constexpr float STATE_F16_UNSCALE = 64.0f;
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
__device__ __forceinline__ float2 unpack_f16x2(uint32_t v) {
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
// as pack_f16x2, values beyond the fp16 range become +-65504 instead of infinity
__device__ __forceinline__ uint32_t pack_f16x2_sat(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
__device__ __forceinline__ uint32_t mul_f16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t fma_f16x2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// tanh of both fp16 halves (the MUFU pipe handles the pair at the rate of two scalar operations)
__device__ __forceinline__ uint32_t tanh_f16x2(uint32_t a) {
    uint32_t d;
    asm("tanh.approx.f16x2 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
// a0 += x.lo * y.lo, a1 += x.hi * y.hi with fp16 factors and fp32 accumulation (mixed-precision FMA of sm_100:
// the product of two fp16 values is exact in fp32)
__device__ __forceinline__ void fma_f32_f16x2(float& a0, float& a1, uint32_t x, uint32_t y) {
    asm("{\n\t.reg .b16 xl, xh, yl, yh;\n\t"
        "mov.b32 {xl, xh}, %2;\n\t"
        "mov.b32 {yl, yh}, %3;\n\t"
        "fma.rn.f32.f16 %0, xl, yl, %0;\n\t"
        "fma.rn.f32.f16 %1, xh, yh, %1;\n\t}"
        : "+f"(a0), "+f"(a1)
        : "r"(x), "r"(y));
}
// the same with bf16 factors
__device__ __forceinline__ void fma_f32_bf16x2(float& a0, float& a1, uint32_t x, uint32_t y) {
    asm("{\n\t.reg .b16 xl, xh, yl, yh;\n\t"
        "mov.b32 {xl, xh}, %2;\n\t"
        "mov.b32 {yl, yh}, %3;\n\t"
        "fma.rn.f32.bf16 %0, xl, yl, %0;\n\t"
        "fma.rn.f32.bf16 %1, xh, yh, %1;\n\t}"
        : "+f"(a0), "+f"(a1)
        : "r"(x), "r"(y));
}
// both fp16 halves converted to bf16 (through fp32, round to nearest)
__device__ __forceinline__ uint32_t f16x2_to_bf16x2(uint32_t v) {
    uint32_t d;
    asm("{\n\t.reg .b16 l, h;\n\t.reg .f32 fl, fh;\n\t"
        "mov.b32 {l, h}, %1;\n\t"
        "cvt.f32.f16 fl, l;\n\t"
        "cvt.f32.f16 fh, h;\n\t"
        "cvt.rn.bf16x2.f32 %0, fh, fl;\n\t}"
        : "=r"(d)
        : "r"(v));
    return d;
}
// both bf16 halves converted to fp16 (values beyond the fp16 range become +-65504)
__device__ __forceinline__ uint32_t bf16x2_to_f16x2_sat(uint32_t v) {
    uint32_t d;
    asm("{\n\t.reg .f32 fl, fh;\n\t"
        "shl.b32 fl, %1, 16;\n\t"
        "and.b32 fh, %1, 0xffff0000;\n\t"
        "cvt.rn.satfinite.f16x2.f32 %0, fh, fl;\n\t}"
        : "=r"(d)
        : "r"(v));
    return d;
}
// Instruction descriptor for kind::f16 with explicit operand formats (0 = fp16, 1 = bf16) and fp32 accumulation.
__device__ __forceinline__ uint32_t umma_idesc_16(int M, int N, int a_mn_major, int b_mn_major, int a_fmt, int b_fmt) {
    return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)a_mn_major << 15) |
           ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// Unpack variants the compiler may not hoist out of a loop: keeping loop-invariant operands packed in registers is
// the point (hoisting the unpack would double their register footprint).
__device__ __forceinline__ float bf16_lo_pinned(uint32_t v) {
    uint32_t r;
    asm volatile("shl.b32 %0, %1, 16;" : "=r"(r) : "r"(v));
    return __uint_as_float(r);
}
__device__ __forceinline__ float bf16_hi_pinned(uint32_t v) {
    uint32_t r;
    asm volatile("and.b32 %0, %1, 0xffff0000;" : "=r"(r) : "r"(v));
    return __uint_as_float(r);
}

}  // namespace ptx
}  // namespace mbema
