// Appearance MLP on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM).
//
// MLPRender_Fea.forward (app/models/mlp_render_fea.py:44-68): 150 -> 128 -> 128 -> 3.  One
// persistent CTA per SM keeps W1 and W2 in shared memory as fp16 in the tensor core's
// K-major "interleaved" (no-swizzle) operand layout and walks tiles of 128 appearance samples.
// A CTA has NSLOT groups of 128 threads; each group owns one tile at a time (thread = sample
// row = TMEM lane) and its own 128 TMEM columns, so that while one group runs its CUDA-core
// phases (positional encoding, bias + ReLU, the 128 -> 3 layer, sigmoid) the other group's
// MMAs occupy the tensor pipe.
//
//   per tile:  build A1[128 x 160] (fp16, optionally hi + lo)      -> smem
//              D = A1 * W1^T   (10 K-steps of tcgen05.mma M128 N128 K16, fp32 accumulate)
//              A2 = relu(D + b1) (fp16, optionally hi + lo)         TMEM -> registers -> smem
//              D = A2 * W2^T   (8 K-steps)
//              rgb = sigmoid(W3 * relu(D + b2) + b3)                TMEM -> registers, fp32
//
// Operand layout (both A and B): element (row r, k) lives at byte  (k / 8) * 2048 + r * 16 +
// (k % 8) * 2; i.e. 8 rows x 16 B form one contiguous 128 B core matrix, row groups are 128 B
// apart (stride byte offset) and the two K halves of one MMA are 2048 B apart (leading byte
// offset).  TA = 2 adds the fp16 rounding residual of the activations as a second MMA per
// K-step (activations then carry ~22 mantissa bits; weights stay single fp16).
//
// Every wait on an mbarrier is bounded; when it expires the kernel raises
// status[GNR_ST_WAIT_EXPIRED], stops taking tiles, frees its TMEM and returns.
#include <cuda_fp16.h>

#include "gnr_internal.cuh"

namespace {

constexpr int HID = 128;
constexpr int APP = 27, FPE = 2, VPE = 2;
constexpr int IN_DIM = APP + 3 + 2 * FPE * APP + 2 * VPE * 3;  // 150
constexpr int K1 = 160, K2 = 128;                              // padded to the MMA K (16)
constexpr int KG1 = K1 / 8, KG2 = K2 / 8;                      // 16-byte K groups
constexpr int ROWS = 128;
constexpr int KG_BYTES = ROWS * 16;                            // 2048: one K group of all rows
constexpr int W1_BYTES = KG1 * KG_BYTES, W2_BYTES = KG2 * KG_BYTES, A_BYTES = KG1 * KG_BYTES;
constexpr int FEAT_STRIDE = 28;
constexpr uint32_t kWaitLimit = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  // K-major, no swizzle: start address, leading byte offset 2048, stride byte offset 128 (all >> 4), version 1
  return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)(KG_BYTES >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) |
         ((uint64_t)1 << 46);
}

// fp16 x fp16 -> fp32, A and B K-major, M = 128, N = 128
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(HID >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);

__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void mma_commit(uint32_t mbar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
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
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, uint32_t parity) {
  for (uint32_t it = 0; it < kWaitLimit; ++it) {
    if (mbar_try_wait(mbar, parity)) return true;
    if (it > 64) __nanosleep(64);
  }
  return false;
}

// One thread of the group waits (bounded) and publishes the outcome; the whole group leaves
// with the same answer, so a group either continues or stops as one.
__device__ __forceinline__ bool group_wait(uint32_t mbar, uint32_t parity, int bar_id, int row, volatile uint32_t* flag) {
  if (row == 0) *flag = mbar_wait_bounded(mbar, parity) ? 1u : 0u;
  asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
  const bool ok = *flag != 0;
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  return ok;
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
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
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

struct TcArgs {
  const float* rays;
  const uint32_t* ids;
  const int32_t* app_index;
  const int32_t* total_ptr;
  long long capacity;
  const float* feat;
  const unsigned char* w_image;  // [W1 fp16 operand image][W2 fp16 operand image]
  const float* w3;
  const float* b1;
  const float* b2;
  const float* b3;
  float* rgb_out;
  int32_t* status;
  int kbits;
};

template <int TA, int NSLOT>
__global__ void __launch_bounds__(NSLOT * 128, 1) mlp_tc_kernel(TcArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* s_w1 = smem;
  unsigned char* s_w2 = s_w1 + W1_BYTES;
  unsigned char* s_a = s_w2 + W2_BYTES;  // [NSLOT][TA][A_BYTES]
  float* s_w3 = reinterpret_cast<float*>(s_a + NSLOT * TA * A_BYTES);
  float* s_b1 = s_w3 + 3 * HID;
  float* s_b2 = s_b1 + HID;
  float* s_b3 = s_b2 + HID;
  uint64_t* s_mbar = reinterpret_cast<uint64_t*>(s_b3 + 4);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_mbar + NSLOT);
  volatile uint32_t* s_flag = s_tmem + 1 + (threadIdx.x >> 7);  // per-group outcome of the last wait

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slot = tid >> 7, row = tid & 127;

  // ---- one-time set-up: weights -> smem, mbarriers, TMEM ---------------------------------------
  {
    const uint4* src = reinterpret_cast<const uint4*>(a.w_image);
    uint4* dst = reinterpret_cast<uint4*>(s_w1);
    for (int i = tid; i < (W1_BYTES + W2_BYTES) / 16; i += NSLOT * 128) dst[i] = src[i];
    for (int i = tid; i < 3 * HID; i += NSLOT * 128) s_w3[i] = a.w3[i];
    for (int i = tid; i < HID; i += NSLOT * 128) {
      s_b1[i] = a.b1[i];
      s_b2[i] = a.b2[i];
    }
    if (tid < 4) s_b3[tid] = a.b3[tid];
    if (tid == 0) {
      for (int s = 0; s < NSLOT; ++s)
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_mbar[s])));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                   "r"((uint32_t)(NSLOT * HID < 32 ? 32 : NSLOT * HID)));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  const uint32_t tmem_base = *s_tmem;
  const uint32_t d_tmem = tmem_base + (uint32_t)(slot * HID);                        // this group's accumulator
  const uint32_t my_taddr = d_tmem + ((uint32_t)((warp & 3) * 32) << 16);            // this warp's lane quarter
  unsigned char* a_hi = s_a + (slot * TA) * A_BYTES;
  unsigned char* a_lo = a_hi + (TA == 2 ? A_BYTES : 0);
  const uint32_t a_hi_addr = smem_u32(a_hi), a_lo_addr = smem_u32(a_lo);
  const uint32_t w1_addr = smem_u32(s_w1), w2_addr = smem_u32(s_w2);
  const uint32_t mbar = smem_u32(&s_mbar[slot]);
  const int bar_id = 1 + slot;  // named barrier of this group (0 is __syncthreads)
  uint32_t parity = 0;

  const long long total = min((long long)*a.total_ptr, a.capacity);
  const long long n_tiles = (total + ROWS - 1) / ROWS;

  for (long long tile = (long long)blockIdx.x * NSLOT + slot; tile < n_tiles; tile += (long long)gridDim.x * NSLOT) {
    const long long j = tile * ROWS + row;
    const bool live = j < total;

    // ---- phase 1: this row of the layer-1 input ---------------------------------------------
    {
      float f[FEAT_STRIDE];
      float view[3] = {0.0f, 0.0f, 0.0f};
      if (live) {
        const float4* fr = reinterpret_cast<const float4*>(a.feat + (size_t)j * FEAT_STRIDE);
#pragma unroll
        for (int q = 0; q < FEAT_STRIDE / 4; ++q) {
          const float4 v = __ldg(fr + q);
          f[4 * q] = v.x;
          f[4 * q + 1] = v.y;
          f[4 * q + 2] = v.z;
          f[4 * q + 3] = v.w;
        }
        const uint32_t ray = __ldg(a.ids + __ldg(a.app_index + j)) >> a.kbits;
        view[0] = __ldg(a.rays + (size_t)ray * 6 + 3);
        view[1] = __ldg(a.rays + (size_t)ray * 6 + 4);
        view[2] = __ldg(a.rays + (size_t)ray * 6 + 5);
      } else {
#pragma unroll
        for (int q = 0; q < FEAT_STRIDE; ++q) f[q] = 0.0f;
      }
      float x[K1];
#pragma unroll
      for (int i = 0; i < APP; ++i) x[i] = f[i];
#pragma unroll
      for (int i = 0; i < 3; ++i) x[APP + i] = view[i];
      // sin/cos of v and 2 v: one accurate sincos, then the double-angle identities
#pragma unroll
      for (int i = 0; i < APP; ++i) {
        float s, c;
        sincosf(f[i], &s, &c);
        x[APP + 3 + 2 * i] = s;
        x[APP + 3 + 2 * i + 1] = 2.0f * s * c;
        x[APP + 3 + 2 * APP + 2 * i] = c;
        x[APP + 3 + 2 * APP + 2 * i + 1] = 1.0f - 2.0f * s * s;
      }
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        float s, c;
        sincosf(view[i], &s, &c);
        x[APP + 3 + 4 * APP + 2 * i] = s;
        x[APP + 3 + 4 * APP + 2 * i + 1] = 2.0f * s * c;
        x[APP + 3 + 4 * APP + 6 + 2 * i] = c;
        x[APP + 3 + 4 * APP + 6 + 2 * i + 1] = 1.0f - 2.0f * s * s;
      }
#pragma unroll
      for (int i = IN_DIM; i < K1; ++i) x[i] = 0.0f;
#pragma unroll
      for (int kg = 0; kg < KG1; ++kg) {
        float g[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] = x[kg * 8 + e];
        store_group<TA>(a_hi, a_lo, kg, row, g);
      }
    }
    proxy_fence();
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");

    // ---- layer 1 MMAs (one thread of the group) ----------------------------------------------
    if (row == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < K1 / 16; ++ks) {
        const uint64_t bd = make_desc(w1_addr + ks * 2 * KG_BYTES);
        mma_f16(d_tmem, make_desc(a_hi_addr + ks * 2 * KG_BYTES), bd, ks > 0 ? 1u : 0u);
        if (TA == 2) mma_f16(d_tmem, make_desc(a_lo_addr + ks * 2 * KG_BYTES), bd, 1u);
      }
      mma_commit(mbar);
    }
    if (!group_wait(mbar, parity, bar_id, row, s_flag)) {
      if (row == 0) atomicExch(a.status + GNR_ST_WAIT_EXPIRED, 1);
      break;
    }
    parity ^= 1;

    // ---- phase 2: A2 = relu(D + b1) -> smem ----------------------------------------------------
#pragma unroll
    for (int cb = 0; cb < HID / 32; ++cb) {
      uint32_t v[32];
      tmem_ld32(my_taddr + cb * 32, v);
#pragma unroll
      for (int g8 = 0; g8 < 4; ++g8) {
        float g[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] = fmaxf(__uint_as_float(v[g8 * 8 + e]) + s_b1[cb * 32 + g8 * 8 + e], 0.0f);
        store_group<TA>(a_hi, a_lo, cb * 4 + g8, row, g);
      }
    }
    tc_fence_before();
    proxy_fence();
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");

    // ---- layer 2 MMAs ---------------------------------------------------------------------------
    if (row == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < K2 / 16; ++ks) {
        const uint64_t bd = make_desc(w2_addr + ks * 2 * KG_BYTES);
        mma_f16(d_tmem, make_desc(a_hi_addr + ks * 2 * KG_BYTES), bd, ks > 0 ? 1u : 0u);
        if (TA == 2) mma_f16(d_tmem, make_desc(a_lo_addr + ks * 2 * KG_BYTES), bd, 1u);
      }
      mma_commit(mbar);
    }
    if (!group_wait(mbar, parity, bar_id, row, s_flag)) {
      if (row == 0) atomicExch(a.status + GNR_ST_WAIT_EXPIRED, 1);
      break;
    }
    parity ^= 1;

    // ---- phase 3: rgb = sigmoid(W3 relu(D + b2) + b3), fp32 on the CUDA cores ------------------
    float o0 = s_b3[0], o1 = s_b3[1], o2 = s_b3[2];
#pragma unroll
    for (int cb = 0; cb < HID / 32; ++cb) {
      uint32_t v[32];
      tmem_ld32(my_taddr + cb * 32, v);
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int c = cb * 32 + e;
        const float h = fmaxf(__uint_as_float(v[e]) + s_b2[c], 0.0f);
        o0 = fmaf(h, s_w3[c], o0);
        o1 = fmaf(h, s_w3[HID + c], o1);
        o2 = fmaf(h, s_w3[2 * HID + c], o2);
      }
    }
    if (live) {
      float* out = a.rgb_out + (size_t)j * 3;
      out[0] = 1.0f / (1.0f + expf(-o0));
      out[1] = 1.0f / (1.0f + expf(-o1));
      out[2] = 1.0f / (1.0f + expf(-o2));
    }
    // the next tile's phase 1 overwrites A and its MMAs overwrite D: order this group's TMEM
    // reads before them
    tc_fence_before();
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
  }

  // ---- teardown -----------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)(NSLOT * HID < 32 ? 32 : NSLOT * HID)));
  }
  (void)lane;
}

// W [n_out = 128][k_real] fp32 -> fp16 operand image [k_groups][128][8]
__global__ void pack_weight_image_kernel(const float* __restrict__ w, __half* __restrict__ img, int k_real, int k_groups) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (kg, n)
  if (i >= k_groups * HID) return;
  int kg = i / HID, n = i - kg * HID;
  __half* dst = img + (size_t)i * 8;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    int k = kg * 8 + e;
    dst[e] = __float2half_rn(k < k_real ? w[(size_t)n * k_real + k] : 0.0f);
  }
}

template <int TA, int NSLOT>
int launch_variant(const GnrModel* m, const TcArgs& args, cudaStream_t st) {
  const size_t smem = (size_t)W1_BYTES + W2_BYTES + (size_t)NSLOT * TA * A_BYTES + (3 * HID + 2 * HID + 4) * sizeof(float) +
                      NSLOT * sizeof(uint64_t) + 32;
  cudaError_t e = cudaFuncSetAttribute(mlp_tc_kernel<TA, NSLOT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  mlp_tc_kernel<TA, NSLOT><<<m->sm_count, NSLOT * 128, smem, st>>>(args);
  return (int)cudaGetLastError();
}

}  // namespace

int gnr_mlp_tc_prepare(GnrModel* m, const float* w1, const float* b1, const float* w2, const float* b2, const float* w3,
                       const float* b3, cudaStream_t st) {
  (void)b1;
  (void)b2;
  (void)w3;
  (void)b3;
  const GnrConfig& c = m->cfg;
  if (c.app_dim != APP || c.fea_pe != FPE || c.view_pe != VPE || c.hidden != HID) {
    gnr_set_error("tensor-core MLP supports app_dim 27, fea_pe 2, view_pe 2, featureC 128 (got %d, %d, %d, %d); use mlp_mode 0",
                  c.app_dim, c.fea_pe, c.view_pe, c.hidden);
    return -1;
  }
  if (m->mlp.tc_image) cudaFree(m->mlp.tc_image);
  m->mlp.tc_image = nullptr;
  m->mlp.tc_image_bytes = (size_t)W1_BYTES + W2_BYTES;
  GNR_CUDA_OK(cudaMalloc(&m->mlp.tc_image, m->mlp.tc_image_bytes));
  __half* img = reinterpret_cast<__half*>(m->mlp.tc_image);
  pack_weight_image_kernel<<<(KG1 * HID + 255) / 256, 256, 0, st>>>(w1, img, IN_DIM, KG1);
  pack_weight_image_kernel<<<(KG2 * HID + 255) / 256, 256, 0, st>>>(w2, img + W1_BYTES / 2, HID, KG2);
  GNR_CUDA_OK(cudaGetLastError());
  return 0;
}

int launch_mlp_tc(const GnrModel* m, const GnrSampleParams& p, const float* rays, char* ws, const GnrWs& L,
                  int64_t max_app, cudaStream_t st) {
  if (!m->mlp.tc_image) {
    gnr_set_error("tensor-core MLP weights were not prepared");
    return -1;
  }
  if (L.feat_stride != FEAT_STRIDE) {
    gnr_set_error("tensor-core MLP expects a feature stride of %d floats", FEAT_STRIDE);
    return -1;
  }
  TcArgs a;
  a.rays = rays;
  a.ids = (const uint32_t*)(ws + L.ids);
  a.app_index = (const int32_t*)(ws + L.app_index);
  a.total_ptr = (const int32_t*)(ws + L.app_offsets) + L.n_rays;
  a.capacity = (long long)max_app;
  a.feat = (const float*)(ws + L.app_feat);
  a.w_image = (const unsigned char*)m->mlp.tc_image;
  a.w3 = m->mlp.w3;
  a.b1 = m->mlp.b1;
  a.b2 = m->mlp.b2;
  a.b3 = m->mlp.b3;
  a.rgb_out = (float*)(ws + L.app_rgb);
  a.status = (int32_t*)(ws + L.status);
  a.kbits = p.kbits;
  if (m->cfg.mlp_mode == 1) return launch_variant<2, 1>(m, a, st);  // activations hi + lo
  if (m->cfg.mlp_mode == 2) return launch_variant<1, 2>(m, a, st);  // single fp16, two tiles in flight
  gnr_set_error("unknown mlp_mode %d", m->cfg.mlp_mode);
  return -1;
}
