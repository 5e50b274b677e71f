// tcgen05 / TMEM / mbarrier helpers and the operand geometry of the appearance network
// (150 -> 128 -> 128 -> 3 behind a 144 -> 27 basis projection), shared by the tensor-core kernels.
#pragma once
#include <cuda_fp16.h>

#include "gnr_internal.cuh"

namespace {

constexpr int HID = 128;
constexpr int APP = 27, FPE = 2, VPE = 2;
constexpr int IN_DIM = APP + 3 + 2 * FPE * APP + 2 * VPE * 3;  // 150
constexpr int K1 = 160, K2 = 144;                              // layer inputs + one constant-1 column for the
                                                               // bias, padded to the MMA K (16)
constexpr int BIAS_COL1 = IN_DIM, BIAS_COL2 = HID;             // where that column sits
constexpr int KG1 = K1 / 8, KG2 = K2 / 8;                      // 16-byte K groups
constexpr int ROWS = 128;
constexpr int KG_BYTES = ROWS * 16;                            // 2048: one K group of all rows
constexpr int NB = 32;                                         // basis outputs padded to the MMA N
constexpr int KGB_BYTES = NB * 16;                             // 512: one K group of the basis operand
constexpr int MAX_K0 = 160;                                    // products per sample the A buffer can hold
constexpr int W1_BYTES = KG1 * KG_BYTES, W2_BYTES = KG2 * KG_BYTES, A_BYTES = KG1 * KG_BYTES;
constexpr int WB_BYTES = (MAX_K0 / 8) * KGB_BYTES;
constexpr int N3 = 16;                                         // layer-3 outputs padded to the smallest MMA N
constexpr int KG3_BYTES = N3 * 16;                             // 256: one K group of the layer-3 operand
constexpr int W3_BYTES = (HID / 8) * KG3_BYTES;                // 4096
constexpr int FEAT_STRIDE = 28;
constexpr int COLS_PER_SLOT = HID + NB;  // D (128) + F (32)
constexpr uint32_t kWaitLimit = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// K-major, no swizzle: start address, leading byte offset, stride byte offset 128 (all >> 4), version 1
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes) {
  return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) |
         ((uint64_t)1 << 46);
}

// fp16 x fp16 -> fp32, A and B K-major, M = 128
constexpr uint32_t kIdescHid = (1u << 4) | ((uint32_t)(HID >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
constexpr uint32_t kIdescBasis = (1u << 4) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
constexpr uint32_t kIdescOut = (1u << 4) | ((uint32_t)(N3 >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);

// `issue` != 0 in exactly one lane (elect_one): the whole warp runs the surrounding loop, so the
// descriptors are computed in warp-uniform code, and the instruction itself is predicated.
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                        uint32_t issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}

// Same, with the A operand in tensor memory: lane = row, one 32-bit column = two consecutive k (fp16).
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                           uint32_t issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}

// One lane of a converged warp.  The MMAs are issued from warp-uniform control flow (a whole warp
// enters, one elected lane issues) with operands derived from warp-uniform values, so that the
// descriptors live in uniform registers; issued from a divergent `if (thread == 0)` every MMA
// first moves its operands there, which costs about 100 cycles per instruction.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(pred));
  return pred;
}

__device__ __forceinline__ void mma_commit(uint32_t mbar, uint32_t issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}\n" ::"r"(mbar), "r"(issue)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ bool mbar_try_wait(uint32_t mbar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t"
      "}"
      : "=r"(ok)
      : "r"(mbar), "r"(parity)
      : "memory");
  return ok != 0;
}

// false if the wait gave up
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, uint32_t parity, uint32_t limit = kWaitLimit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait(mbar, parity)) return true;
    if (it > 64) __nanosleep(64);
  }
  return false;
}

// One thread of the group waits (bounded) and publishes the outcome; the whole group leaves
// with the same answer, so a group either continues or stops as one.
__device__ __forceinline__ bool group_wait(uint32_t mbar, uint32_t parity, int bar_id, int row, volatile uint32_t* flag,
                                           uint32_t limit = kWaitLimit, int group_threads = 128) {
  if (row == 0) *flag = mbar_wait_bounded(mbar, parity, limit) ? 1u : 0u;
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(group_threads) : "memory");
  const bool ok = *flag != 0;
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  return ok;
}

// Bulk async copy global -> shared, completion counted in bytes on an mbarrier.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t mbar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(mbar)
               : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32"
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
      " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&v)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0],"
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16,"
      " %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
      "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
      "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0],"
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};\n" ::"r"(taddr), "r"(v[0]),
               "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// sin and cos for operands that are about to be rounded to fp16 (relative step 4.9e-4): the
// hardware approximations, which reduce the argument themselves (absolute error about 1e-6 for
// the |x| of a few units that features and view directions have).
__device__ __forceinline__ void sincos_reduced(float x, float& s, float& c) { __sincosf(x, &s, &c); }

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// max(x, 0) and the conversion to two fp16 in one instruction; `a` lands in the low half
__device__ __forceinline__ uint32_t pack_h2_relu(float a, float b) {
  uint32_t d;
  asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
  return d;
}

// Store 8 consecutive-k values of one row as fp16 (and, with TA == 2, their rounding residuals).
template <int TA>
__device__ __forceinline__ void store_group(unsigned char* a_hi, unsigned char* a_lo, int kg, int row, const float (&x)[8]) {
  uint4 hi;
  hi.x = pack_h2(x[0], x[1]);
  hi.y = pack_h2(x[2], x[3]);
  hi.z = pack_h2(x[4], x[5]);
  hi.w = pack_h2(x[6], x[7]);
  *reinterpret_cast<uint4*>(a_hi + kg * KG_BYTES + row * 16) = hi;
  if (TA == 2) {
    float r[8];
    const __half2* hp = reinterpret_cast<const __half2*>(&hi);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f = __half22float2(hp[e]);
      r[2 * e] = x[2 * e] - f.x;
      r[2 * e + 1] = x[2 * e + 1] - f.y;
    }
    uint4 lo;
    lo.x = pack_h2(r[0], r[1]);
    lo.y = pack_h2(r[2], r[3]);
    lo.z = pack_h2(r[4], r[5]);
    lo.w = pack_h2(r[6], r[7]);
    *reinterpret_cast<uint4*>(a_lo + kg * KG_BYTES + row * 16) = lo;
  }
}

}  // namespace
