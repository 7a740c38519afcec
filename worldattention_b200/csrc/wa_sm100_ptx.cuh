// PTX wrappers and softmax arithmetic shared by the tcgen05 kernels (sm_100a): mbarriers with bounded
// waits, TMA tile loads and stores, tcgen05.mma / ld / st / commit, tensor-memory shapes, exp2 on the
// FMA pipe.  Everything here is device code; nothing allocates.
#pragma once
#include <cuda.h>

#include "wa_common.cuh"

namespace wa {
namespace sm100 {

constexpr int TILE = 128;            // query rows, key tokens and head_dim of one tile
constexpr int HALF = 64;             // key tokens per softmax / MMA pipeline step
constexpr int HALF_BYTES = TILE * 64 * 2;   // one TMA box: 128 rows x 64 bf16 (128 B per row)
constexpr int TILE_BYTES = 2 * HALF_BYTES;  // 32 KB
constexpr long long WAIT_CYCLES = 4000000000ll;   // bound of every mbarrier wait (about two seconds)

// ---- PTX wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival for the whole warp: every lane has finished (and fenced) its part before lane 0 signals.
__device__ __forceinline__ void warp_arrive(uint64_t *bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"   // %3: the thread may sleep this many ns
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(2000u) : "memory");
    return ok != 0;
}
// Same with a caller-chosen sleep limit (for a thread that watches two barriers).
__device__ __forceinline__ bool mbar_try_wait_ns(uint64_t *bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// Non-blocking test of a barrier phase.
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Where a wait that ran out leaves its site code: the flag in the call's workspace and, when the caller gave one,
// a word the host can read without a copy (page-locked host memory).
struct FailSink {
    int *flag;
    int *mirror;
};
__device__ __forceinline__ void report_failure(const FailSink &sink, int code) {
    atomicExch(sink.flag, code);
    if (sink.mirror) {
        *reinterpret_cast<volatile int *>(sink.mirror) = code;
        __threadfence_system();
    }
}
// Bounded wait.  Returns false after the abort flag is raised or the time budget is spent.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, const FailSink &sink,
                                          int code) {
    if (mbar_test(bar, parity)) return true;   // the common case: the phase is over already
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_CYCLES) {
            *abort_flag = 1;
            report_failure(sink, code);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, const void *src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, const void *src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}

#define TMEM_LD32(taddr, r)                                                                                          \
    asm volatile(                                                                                                    \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                                    \
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                                    \
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"                    \
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),            \
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),      \
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),    \
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])     \
        : "r"(taddr) : "memory")

#define TMEM_LD16(taddr, r)                                                                                          \
    asm volatile(                                                                                                    \
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "                                                                    \
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"                             \
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),            \
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])       \
        : "r"(taddr) : "memory")

#define TMEM_ST16(taddr, r)                                                                                          \
    asm volatile(                                                                                                    \
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "                                                              \
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"                                   \
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),        \
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory")

#define TMEM_ST32(taddr, r)                                                                                          \
    asm volatile(                                                                                                    \
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "                                                              \
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "                                   \
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"                           \
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),        \
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),              \
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),            \
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory")

// Quad-row shapes: a 16-row group of lanes is read so that thread t holds rows t/4 and t/4+8 and, per 8-column step j,
// the column pair 8j + 2(t%4), +1 of each (registers 4j..4j+3: row A pair, row B pair) -- a row lives in one quad.
// The 16x128b store is the matching shape for 32-bit words: registers 2j, 2j+1 = word 4j + t%4 of row A, row B.
#define TMEM_LDQ64(taddr, r) \
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];" \
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63]) \
        : "r"(taddr) : "memory")
#define TMEM_LDQ16(taddr, r) \
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];" \
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]) \
        : "r"(taddr) : "memory")
#define TMEM_STQ16(taddr, r) \
    asm volatile("tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" \
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory")
#define TMEM_STP32(taddr, r) \
    asm volatile("tcgen05.st.sync.aligned.16x128b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" \
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory")

#define TMEM_STP16(taddr, r) \
    asm volatile("tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" \
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory")

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Shared-memory matrix descriptor, 128-byte swizzle.  `lbo`, `sbo` in bytes.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;   // descriptor version of this architecture
    d |= (uint64_t)2 << 61;   // 128-byte swizzle
    return d;
}

// kind::f16 instruction descriptor: bf16 x bf16 -> f32, M = N = 128; `b_mn_major` for the V operand.
__host__ __device__ constexpr uint32_t instr_desc(bool b_mn_major, int n) {
    return (1u << 4)                 // D format f32
           | (1u << 7)               // A format bf16
           | (1u << 10)              // B format bf16
           | ((b_mn_major ? 1u : 0u) << 16)
           | ((uint32_t)(n >> 3) << 17)
           | ((uint32_t)(TILE >> 4) << 24);
}

// Softmax arithmetic.  It runs on pairs of columns with the packed float32x2 instructions of this architecture (one
// issue slot for two results).  2^x on the FMA pipe: split x into round(x) + f, f in [-0.5, 0.5], evaluate a
// cubic for 2^f and add round(x) to the exponent field; relative error < 2^-10, below the bf16 rounding of P.
// The special-function unit (16 results per clock per SM) is the narrowest pipe of the softmax, so every
// POLY_EVERY-th pair of columns takes the polynomial instead.
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
    x.x = fmaxf(x.x, -125.0f);
    x.y = fmaxf(x.y, -125.0f);
    const float2 magic = make_float2(12582912.0f, 12582912.0f);   // 1.5 * 2^23: the integer part of x lands in the low mantissa bits
    const float2 t = __fadd2_rn(x, magic);
    const float2 f = __fadd2_rn(x, __fadd2_rn(magic, make_float2(-t.x, -t.y)));   // x - (t - magic)
    float2 q = __ffma2_rn(f, make_float2(0.0555041f, 0.0555041f), make_float2(0.2402265f, 0.2402265f));
    q = __ffma2_rn(q, f, make_float2(0.6931472f, 0.6931472f));
    q = __ffma2_rn(q, f, make_float2(1.0f, 1.0f));
    return make_float2(__uint_as_float(__float_as_uint(q.x) + (__float_as_uint(t.x) << 23)),
                       __uint_as_float(__float_as_uint(q.y) + (__float_as_uint(t.y) << 23)));
}
#ifndef WA_POLY_EVERY
#define WA_POLY_EVERY 4
#endif
constexpr int POLY_EVERY = WA_POLY_EVERY;


// One 8-column step of a quad-row tile: this thread's column pair of row A (x0, x1) and of row B (x2, x3)
// -> probabilities, packed to one bf16 pair per row; row sums accumulate in accA / accB (packed float32x2).
template <bool POLY, bool MASKED>
__device__ __forceinline__ void exp_step(uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3, float2 sc, float2 nmA, float2 nmB,
                                         float2 &accA, float2 &accB, uint32_t &pkA, uint32_t &pkB, int col, int valid) {
    const float2 xa = __ffma2_rn(make_float2(__uint_as_float(x0), __uint_as_float(x1)), sc, nmA);
    const float2 xb = __ffma2_rn(make_float2(__uint_as_float(x2), __uint_as_float(x3)), sc, nmB);
    float2 pa, pb;
    if (POLY) {
        pa = ex2_poly2(xa);
        pb = ex2_poly2(xb);
    } else {
        pa = make_float2(ex2(xa.x), ex2(xa.y));
        pb = make_float2(ex2(xb.x), ex2(xb.y));
    }
    if (MASKED) {
        if (col >= valid) pa.x = pb.x = 0.f;
        if (col + 1 >= valid) pa.y = pb.y = 0.f;
    }
    accA = __fadd2_rn(accA, pa);
    accB = __fadd2_rn(accB, pb);
    __nv_bfloat162 ha = __floats2bfloat162_rn(pa.x, pa.y), hb = __floats2bfloat162_rn(pb.x, pb.y);
    pkA = *reinterpret_cast<uint32_t *>(&ha);
    pkB = *reinterpret_cast<uint32_t *>(&hb);
}

__device__ __forceinline__ float quad_max(float x) {
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
    return fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
}
__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    return x + __shfl_xor_sync(0xffffffffu, x, 2);
}

struct Params {
    int B, H, Lq, Lkv, Lc, Nq, Nkv;
    int blk;       // routing block size: 128, or 64 (a work item is then a 64-row query block in a 128-row tile whose
                   // upper rows are computed and dropped, and a key tile holds two selected 64-token blocks)
    int n_items;
    const int32_t *index;   // [B,H,Nq,Nkv]
    const int32_t *num;     // [B,H,Nq]
    const int32_t *order;   // [n_items] work order (heaviest first)
    int *work_counter;
    int *error_flag;
    int *status_mirror;     // optional host-visible copy of the failure code (see wa_hsa_params::status_mirror)
    __nv_bfloat16 *out;
    long long osb, osl, osh;
    const float *gate_bias;   // [128] or null
    int has_gate;             // 0: gate = sigmoid(q)
    const __nv_bfloat16 *q;   // for the no-gate path
    long long qsb, qsl, qsh;
    float scale_log2;         // D^-1/2 * log2(e)
    // partial-output mode (KV-sharded multi-GPU): normalised per-branch outputs + natural-log LSE
    float *part_sparse, *part_linear;   // float32 or null: vector of (b, token, head) at ((b * Lq + token) * H + head) * part_stride
    float *lse_sparse, *lse_linear;     // float32: value of (b, head, token) at b * lse_sb + head * lse_sh + token * lse_st
    long long part_stride, lse_sb, lse_sh, lse_st;
    // partial outputs stored into peer ranks' buffers (see wa_hsa_params::peer_rows); peer_rows == 0: off
    int lse_packed;
    int peer_rows, peer_self;
    long long peer_delta[8];
};

struct ItemDesc {
    int item;    // (b*H + h)*Nq + qb, or -1: no more work
    int n_sel;   // selected key blocks of this item
};

}  // namespace sm100
}  // namespace wa
