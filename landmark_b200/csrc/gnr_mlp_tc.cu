// Basis projection + appearance MLP on the 5th-generation tensor cores (tcgen05.mma with
// accumulators in tensor memory), one kernel.
//
// compute_appfeature's Linear(144 -> 27) (app/models/gridnerf_sequential.py:678,864-871) and
// MLPRender_Fea.forward (app/models/mlp_render_fea.py:44-68): 150 -> 128 -> 128 -> 3, sigmoid.
//
// One persistent CTA per SM keeps the basis matrix, W1 and W2 in shared memory as fp16 in the
// tensor core's K-major "interleaved" (no-swizzle) operand layout and walks tiles of 128
// appearance samples.  A CTA has NSLOT groups of 128 threads; a group owns one tile at a time
// (thread = sample row = TMEM lane), its own operand buffer and its own 160 TMEM columns, so
// while one group runs its CUDA-core phases another group's MMAs occupy the tensor pipe.
//
//   per tile:  A0[128 x 144] fp16 plane x line products, written by the gather kernel in
//              operand layout, arrive by one bulk async copy (cp.async.bulk -> mbarrier)
//              F  = A0 * Wb^T           (9 K-steps of tcgen05.mma M128 N32 K16, fp32 accumulate)
//              A1 = [F, view, sin/cos(F 2^f), sin/cos(view 2^f)]      TMEM -> registers -> smem
//              D  = A1 * W1^T           (10 K-steps, M128 N128 K16)
//              A2 = relu(D + b1)                                      TMEM -> registers -> smem
//              D  = A2 * W2^T           (8 K-steps)
//              rgb = sigmoid(W3 relu(D + b2) + b3)                    TMEM -> registers, fp32
//
// Biases ride in the MMAs: every layer input carries a constant 1 in its first padding column
// (column 150 of layer 1, column 128 of layer 2) and the weight image holds the bias there, so
// the epilogues only apply ReLU, which the fp16 conversion does itself (cvt.rn.relu.f16x2.f32).
//
// Operand layout (A and B alike): element (row r, k) at byte (k / 8) * LBO + r * 16 + (k % 8) * 2:
// 8 rows x 16 B form one contiguous 128 B core matrix, row groups are 128 B apart (stride byte
// offset), the two K halves of one MMA are LBO = rows * 16 bytes apart (leading byte offset).
// TA = 2 carries the fp16 rounding residual of every activation (and product) as a second
// operand and a second MMA per K-step (activations then hold ~22 mantissa bits; weights stay
// single fp16).
//
// Every wait on an mbarrier is bounded; when one expires the group raises
// status[GNR_ST_WAIT_EXPIRED], stops taking tiles, and the CTA frees its TMEM and returns.
#include "gnr_tc.cuh"

namespace {

struct TcArgs {
  GnrCoords crd;
  const float* feat_in;           // BASIS == false: features from the CUDA-core gather
  float* feat_out;                // BASIS == true: optional copy of the projected features
  const unsigned char* prod_hi;   // BASIS == true: fp16 product tiles in operand layout
  const unsigned char* prod_lo;
  int tile_bytes;                 // bytes of one product tile (k0 / 8 * 2048)
  int k0;                         // products per sample
  const unsigned char* w_image;   // [basis fp16 operand image (WB_BYTES)][W1 image][W2 image][W3 image]
  const float* w3;
  const float* b1;
  const float* b2;
  const float* b3;
  float* rgb_out;
  int32_t* status;
  int kbits;
  int basis_only;                 // stop after the projection: feat_out receives F and nothing else runs
  uint32_t wait_limit;            // polls a bounded wait may take
  int debug_skip_copy;            // test hook: group 0 of CTA 0 never starts the copy of its first tile
};

template <int TA, int NSLOT, bool BASIS>
__global__ void __launch_bounds__(NSLOT * 128, 1) mlp_tc_kernel(TcArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* s_wb = smem;
  unsigned char* s_w1 = s_wb + WB_BYTES;
  unsigned char* s_w2 = s_w1 + W1_BYTES;
  unsigned char* s_w3h = s_w2 + W2_BYTES;  // layer 3 as an fp16 operand (used when L3TC)
  unsigned char* s_a = s_w3h + W3_BYTES;   // [NSLOT][TA][A_BYTES]
  float* s_w3 = reinterpret_cast<float*>(s_a + NSLOT * TA * A_BYTES);
  float* s_b1 = s_w3 + 3 * HID;
  float* s_b2 = s_b1 + HID;
  float* s_b3 = s_b2 + HID;
  uint64_t* s_mbar = reinterpret_cast<uint64_t*>(s_b3 + 4);  // [NSLOT][2]: MMA completion, bulk-copy completion
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_mbar + 2 * NSLOT);
  volatile uint32_t* s_flag = s_tmem + 1;  // [NSLOT] per-group outcome of the last wait (indexed below)

  constexpr uint32_t kTmemCols = (NSLOT * COLS_PER_SLOT <= 256) ? 256u : 512u;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int warp_u = __shfl_sync(0xffffffffu, tid >> 5, 0);  // the same number, known to be warp-uniform
  const int slot = warp_u >> 2, row = tid & 127;
  const bool lead_warp = (warp_u & 3) == 0;                  // the warp of a group that issues its MMAs

  // ---- one-time set-up: weights -> smem, mbarriers, TMEM ---------------------------------------
  {
    const uint4* src = reinterpret_cast<const uint4*>(a.w_image);
    uint4* dst = reinterpret_cast<uint4*>(s_wb);
    for (int i = tid; i < (WB_BYTES + W1_BYTES + W2_BYTES + W3_BYTES) / 16; i += NSLOT * 128) dst[i] = src[i];
    for (int i = tid; i < 3 * HID; i += NSLOT * 128) s_w3[i] = a.w3[i];
    for (int i = tid; i < HID; i += NSLOT * 128) {
      s_b1[i] = a.b1[i];
      s_b2[i] = a.b2[i];
    }
    if (tid < 4) s_b3[tid] = a.b3[tid];
    if (tid == 0) {
      for (int s = 0; s < 2 * NSLOT; ++s)
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_mbar[s])));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                   "r"(kTmemCols));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *s_tmem, 0);  // (broadcast: warp-uniform for the compiler)
  const uint32_t d_tmem = tmem_base + (uint32_t)(slot * COLS_PER_SLOT);     // this group's D accumulator
  const uint32_t f_tmem = d_tmem + HID;                                     // this group's feature accumulator
  const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;              // this warp's TMEM lane quarter
  unsigned char* a_hi = s_a + (slot * TA) * A_BYTES;
  unsigned char* a_lo = a_hi + (TA == 2 ? A_BYTES : 0);
  const uint32_t a_hi_addr = smem_u32(a_hi), a_lo_addr = smem_u32(a_lo);
  const uint32_t wb_addr = smem_u32(s_wb), w1_addr = smem_u32(s_w1), w2_addr = smem_u32(s_w2), w3_addr = smem_u32(s_w3h);
  constexpr bool L3TC = (TA == 1);  // layer 3 on the tensor cores too (fp16 operands); TA == 2 keeps it in fp32
  const uint32_t mbar = smem_u32(&s_mbar[2 * slot]), tbar = smem_u32(&s_mbar[2 * slot + 1]);
  const int bar_id = 1 + slot;  // named barrier of this group (0 is __syncthreads)
  s_flag += slot;
  uint32_t parity = 0, tparity = 0;
  bool copy_pending = false;

  const long long total = min(a.crd.total_ptr ? (long long)*a.crd.total_ptr : a.crd.total_direct, a.crd.capacity);
  const long long n_tiles = (total + ROWS - 1) / ROWS;
  const long long tile_stride = (long long)gridDim.x * NSLOT;
  const uint32_t copy_bytes = (uint32_t)a.tile_bytes;

  auto start_copy = [&](long long t) {
    // one thread: announce the bytes, then start the copies of the tile's operand image(s)
    mbar_expect_tx(tbar, copy_bytes * TA);
    bulk_load(a_hi_addr, a.prod_hi + (size_t)t * copy_bytes, copy_bytes, tbar);
    if (TA == 2) bulk_load(a_lo_addr, a.prod_lo + (size_t)t * copy_bytes, copy_bytes, tbar);
  };

  long long tile = (long long)blockIdx.x * NSLOT + slot;
  const bool skip_first_copy = a.debug_skip_copy != 0 && blockIdx.x == 0 && slot == 0;
  if (BASIS && tile < n_tiles) {
    if (row == 0 && !skip_first_copy) start_copy(tile);
    copy_pending = !skip_first_copy;
  }

  for (; tile < n_tiles; tile += tile_stride) {
    const long long j = tile * ROWS + row;
    const bool live = j < total;
    float f[32];

    if (BASIS) {
      // ---- phase 0: F = A0 * Wb^T ---------------------------------------------------------------
      const bool arrived = group_wait(tbar, tparity, bar_id, row, s_flag, a.wait_limit);
      if (!arrived) {
        if (row == 0) atomicExch(a.status + GNR_ST_WAIT_EXPIRED, 1);
        break;
      }
      copy_pending = false;
      tparity ^= 1;
      if (lead_warp) {
        const uint32_t leader = elect_one();
        const int ksteps = a.k0 >> 4;
#pragma unroll
        for (int ks = 0; ks < MAX_K0 / 16; ++ks) {
          if (ks < ksteps) {
            const uint64_t bd = make_desc(wb_addr + ks * 2 * KGB_BYTES, KGB_BYTES);
            mma_f16(f_tmem, make_desc(a_hi_addr + ks * 2 * KG_BYTES, KG_BYTES), bd, kIdescBasis, ks > 0 ? 1u : 0u, leader);
            if (TA == 2) mma_f16(f_tmem, make_desc(a_lo_addr + ks * 2 * KG_BYTES, KG_BYTES), bd, kIdescBasis, 1u, leader);
          }
        }
        mma_commit(mbar, leader);
        __syncwarp();
      }
      if (!group_wait(mbar, parity, bar_id, row, s_flag, a.wait_limit)) {
        if (row == 0) atomicExch(a.status + GNR_ST_WAIT_EXPIRED, 1);
        break;
      }
      parity ^= 1;
      uint32_t v[32];
      tmem_ld32(f_tmem + lane_off, v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
      if (a.feat_out != nullptr && live) {
        float4* fo = reinterpret_cast<float4*>(a.feat_out + (size_t)j * FEAT_STRIDE);
#pragma unroll
        for (int q = 0; q < FEAT_STRIDE / 4; ++q) fo[q] = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
      }
      if (a.basis_only) {
        // partial projection for channel-parallel rendering: the operand buffer is free as soon as
        // the basis MMAs have completed, so the next tile's products can come in right away
        if (tile + tile_stride < n_tiles) {
          if (row == 0) start_copy(tile + tile_stride);
          copy_pending = true;
        }
        tc_fence_before();  // F was read from tensor memory; the next tile's MMAs overwrite it
        continue;
      }
    } else {
      if (live) {
        const float4* fr = reinterpret_cast<const float4*>(a.feat_in + (size_t)j * FEAT_STRIDE);
#pragma unroll
        for (int q = 0; q < FEAT_STRIDE / 4; ++q) {
          const float4 v = __ldg(fr + q);
          f[4 * q] = v.x;
          f[4 * q + 1] = v.y;
          f[4 * q + 2] = v.z;
          f[4 * q + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int q = 0; q < FEAT_STRIDE; ++q) f[q] = 0.0f;
      }
    }

    // ---- phase 1: this row of the layer-1 input ---------------------------------------------
    {
      float view[3] = {0.0f, 0.0f, 0.0f};
      if (BASIS) {
        // the gather kernel left the view direction in the k group after the products (hi + lo fp16)
        const uint4 vv = *reinterpret_cast<const uint4*>(a_hi + (a.k0 >> 3) * KG_BYTES + row * 16);
        const float2 p0 = __half22float2(*reinterpret_cast<const __half2*>(&vv.x));
        const float2 p1 = __half22float2(*reinterpret_cast<const __half2*>(&vv.y));
        const float2 p2 = __half22float2(*reinterpret_cast<const __half2*>(&vv.z));
        if (live) {
          view[0] = p0.x + p1.y;
          view[1] = p0.y + p2.x;
          view[2] = p1.x + p2.y;
        }
      } else if (live) {
        const float* vsrc;
        if (a.crd.view_direct) {
          vsrc = a.crd.view_direct + (size_t)j * a.crd.point_stride;
        } else {
          const uint32_t ray = __ldg(a.crd.ids + (a.crd.index ? (long long)__ldg(a.crd.index + j) : j)) >> a.kbits;
          vsrc = a.crd.rays + (size_t)ray * 6 + 3;
        }
        view[0] = __ldg(vsrc + 0);
        view[1] = __ldg(vsrc + 1);
        view[2] = __ldg(vsrc + 2);
      }
      float x[K1];
#pragma unroll
      for (int i = 0; i < APP; ++i) x[i] = f[i];
#pragma unroll
      for (int i = 0; i < 3; ++i) x[APP + i] = view[i];
      // sin/cos of v and 2 v: one sincos, then the double-angle identities
#pragma unroll
      for (int i = 0; i < APP; ++i) {
        float s, c;
        sincos_reduced(f[i], s, c);
        x[APP + 3 + 2 * i] = s;
        x[APP + 3 + 2 * i + 1] = 2.0f * s * c;
        x[APP + 3 + 2 * APP + 2 * i] = c;
        x[APP + 3 + 2 * APP + 2 * i + 1] = 1.0f - 2.0f * s * s;
      }
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        float s, c;
        sincos_reduced(view[i], s, c);
        x[APP + 3 + 4 * APP + 2 * i] = s;
        x[APP + 3 + 4 * APP + 2 * i + 1] = 2.0f * s * c;
        x[APP + 3 + 4 * APP + 6 + 2 * i] = c;
        x[APP + 3 + 4 * APP + 6 + 2 * i + 1] = 1.0f - 2.0f * s * s;
      }
      x[BIAS_COL1] = 1.0f;  // multiplies the b1 column of the W1 image
#pragma unroll
      for (int i = IN_DIM + 1; i < K1; ++i) x[i] = 0.0f;
#pragma unroll
      for (int kg = 0; kg < KG1; ++kg) {
        float g[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] = x[kg * 8 + e];
        store_group<TA>(a_hi, a_lo, kg, row, g);
      }
    }
    tc_fence_before();
    proxy_fence();
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");

    // ---- layer 1 MMAs (one thread of the group) ----------------------------------------------
    if (lead_warp) {
      tc_fence_after();
      const uint32_t leader = elect_one();
#pragma unroll
      for (int ks = 0; ks < K1 / 16; ++ks) {
        const uint64_t bd = make_desc(w1_addr + ks * 2 * KG_BYTES, KG_BYTES);
        mma_f16(d_tmem, make_desc(a_hi_addr + ks * 2 * KG_BYTES, KG_BYTES), bd, kIdescHid, ks > 0 ? 1u : 0u, leader);
        if (TA == 2) mma_f16(d_tmem, make_desc(a_lo_addr + ks * 2 * KG_BYTES, KG_BYTES), bd, kIdescHid, 1u, leader);
      }
      mma_commit(mbar, leader);
      __syncwarp();
    }
    if (!group_wait(mbar, parity, bar_id, row, s_flag, a.wait_limit)) {
      if (row == 0) atomicExch(a.status + GNR_ST_WAIT_EXPIRED, 1);
      break;
    }
    parity ^= 1;

    // ---- phase 2: A2 = relu(D) -> smem (D already holds the bias; two TMEM loads per wait) -------
#pragma unroll
    for (int cb = 0; cb < HID / 64; ++cb) {
      uint32_t v[64];
      tmem_ld32(d_tmem + lane_off + cb * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
      tmem_ld32(d_tmem + lane_off + cb * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
      tmem_ld_wait();
#pragma unroll
      for (int g8 = 0; g8 < 8; ++g8) {
        if (TA == 1) {
          uint4 hi;
          hi.x = pack_h2_relu(__uint_as_float(v[g8 * 8 + 0]), __uint_as_float(v[g8 * 8 + 1]));
          hi.y = pack_h2_relu(__uint_as_float(v[g8 * 8 + 2]), __uint_as_float(v[g8 * 8 + 3]));
          hi.z = pack_h2_relu(__uint_as_float(v[g8 * 8 + 4]), __uint_as_float(v[g8 * 8 + 5]));
          hi.w = pack_h2_relu(__uint_as_float(v[g8 * 8 + 6]), __uint_as_float(v[g8 * 8 + 7]));
          *reinterpret_cast<uint4*>(a_hi + (cb * 8 + g8) * KG_BYTES + row * 16) = hi;
        } else {
          float g[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) g[e] = fmaxf(__uint_as_float(v[g8 * 8 + e]), 0.0f);
          store_group<TA>(a_hi, a_lo, cb * 8 + g8, row, g);
        }
      }
    }
    {
      // the constant-1 column (input 128) and the padding of the last K-step
      const float one[8] = {1.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
      const float zero[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
      store_group<TA>(a_hi, a_lo, HID / 8, row, one);
      store_group<TA>(a_hi, a_lo, HID / 8 + 1, row, zero);
    }
    tc_fence_before();
    proxy_fence();
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");

    // ---- layer 2 MMAs ---------------------------------------------------------------------------
    if (lead_warp) {
      tc_fence_after();
      const uint32_t leader = elect_one();
#pragma unroll
      for (int ks = 0; ks < K2 / 16; ++ks) {
        const uint64_t bd = make_desc(w2_addr + ks * 2 * KG_BYTES, KG_BYTES);
        mma_f16(d_tmem, make_desc(a_hi_addr + ks * 2 * KG_BYTES, KG_BYTES), bd, kIdescHid, ks > 0 ? 1u : 0u, leader);
        if (TA == 2) mma_f16(d_tmem, make_desc(a_lo_addr + ks * 2 * KG_BYTES, KG_BYTES), bd, kIdescHid, 1u, leader);
      }
      mma_commit(mbar, leader);
      __syncwarp();
    }
    if (!group_wait(mbar, parity, bar_id, row, s_flag, a.wait_limit)) {
      if (row == 0) atomicExch(a.status + GNR_ST_WAIT_EXPIRED, 1);
      break;
    }
    parity ^= 1;
    // the operand buffer is free again: fetch the next tile's products while phase 3 runs
    if (BASIS && tile + tile_stride < n_tiles) {
      if (row == 0) start_copy(tile + tile_stride);
      copy_pending = true;
    }

    float o0, o1, o2;
    if (L3TC) {
      // ---- phase 3 (tensor cores): relu(D) goes back into tensor memory as packed fp16 pairs, over the
      // columns of D this thread has already read (64 columns hold k = 0..127), and is the A operand
      // of 8 more MMAs (N = 16, 3 real outputs) whose accumulator reuses the feature columns.
#pragma unroll
      for (int cb = 0; cb < HID / 64; ++cb) {
        uint32_t v[64];
        tmem_ld32(d_tmem + lane_off + cb * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
        tmem_ld32(d_tmem + lane_off + cb * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
        tmem_ld_wait();
        uint32_t h[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) h[e] = pack_h2_relu(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
        tmem_st32(d_tmem + lane_off + cb * 32, h);
      }
      tmem_st_wait();
      tc_fence_before();
      asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
      if (lead_warp) {
        tc_fence_after();
        const uint32_t leader = elect_one();
#pragma unroll
        for (int ks = 0; ks < HID / 16; ++ks)
          mma_f16_ts(f_tmem, d_tmem + ks * 8, make_desc(w3_addr + ks * 2 * KG3_BYTES, KG3_BYTES), kIdescOut, ks > 0 ? 1u : 0u, leader);
        mma_commit(mbar, leader);
        __syncwarp();
      }
      if (!group_wait(mbar, parity, bar_id, row, s_flag, a.wait_limit)) {
        if (row == 0) atomicExch(a.status + GNR_ST_WAIT_EXPIRED, 1);
        break;
      }
      parity ^= 1;
      uint32_t r[4];
      tmem_ld4(f_tmem + lane_off, r);
      tmem_ld_wait();
      o0 = s_b3[0] + __uint_as_float(r[0]);
      o1 = s_b3[1] + __uint_as_float(r[1]);
      o2 = s_b3[2] + __uint_as_float(r[2]);
    } else {
      // ---- phase 3 (CUDA cores): rgb = sigmoid(W3 relu(D) + b3) in fp32, packed fp32x2 FMAs ----------
      float2 p0 = make_float2(0.0f, 0.0f), p1 = p0, p2 = p0;
#pragma unroll
      for (int cb = 0; cb < HID / 64; ++cb) {
        uint32_t v[64];
        tmem_ld32(d_tmem + lane_off + cb * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
        tmem_ld32(d_tmem + lane_off + cb * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
        tmem_ld_wait();
#pragma unroll
        for (int e4 = 0; e4 < 16; ++e4) {
          const int c = cb * 64 + e4 * 4;
          const float4 wr = *reinterpret_cast<const float4*>(s_w3 + c);
          const float4 wg = *reinterpret_cast<const float4*>(s_w3 + HID + c);
          const float4 wb = *reinterpret_cast<const float4*>(s_w3 + 2 * HID + c);
          const float2 ha = make_float2(fmaxf(__uint_as_float(v[e4 * 4 + 0]), 0.0f), fmaxf(__uint_as_float(v[e4 * 4 + 1]), 0.0f));
          const float2 hb = make_float2(fmaxf(__uint_as_float(v[e4 * 4 + 2]), 0.0f), fmaxf(__uint_as_float(v[e4 * 4 + 3]), 0.0f));
          p0 = __ffma2_rn(hb, make_float2(wr.z, wr.w), __ffma2_rn(ha, make_float2(wr.x, wr.y), p0));
          p1 = __ffma2_rn(hb, make_float2(wg.z, wg.w), __ffma2_rn(ha, make_float2(wg.x, wg.y), p1));
          p2 = __ffma2_rn(hb, make_float2(wb.z, wb.w), __ffma2_rn(ha, make_float2(wb.x, wb.y), p2));
        }
      }
      o0 = s_b3[0] + (p0.x + p0.y);
      o1 = s_b3[1] + (p1.x + p1.y);
      o2 = s_b3[2] + (p2.x + p2.y);
    }
    if (live) {
      float* out = a.rgb_out + (size_t)j * 3;
      out[0] = 1.0f / (1.0f + expf(-o0));
      out[1] = 1.0f / (1.0f + expf(-o1));
      out[2] = 1.0f / (1.0f + expf(-o2));
    }
    // the next tile's MMAs overwrite F and D: order this group's TMEM reads before the syncs
    // that precede them
    tc_fence_before();
    if (!BASIS) asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
  }

  // ---- teardown -----------------------------------------------------------------------------------
  if (copy_pending) {
    // a group that stopped early still has a bulk copy in flight into its operand buffer
    group_wait(tbar, tparity, bar_id, row, s_flag, a.wait_limit);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols));
  }
}

// W [n_out][k_real] fp32 -> fp16 operand image [k_groups][n_rows][8]; rows >= n_out and
// columns >= k_real are zero, except column `bias_col`, which takes `bias`.  `k_map_c`/`k_map_cp` translate a padded product index
// (pair * cp + c) into the column of the unpadded matrix; pass 0 for a plain matrix.
__global__ void pack_weight_image_kernel(const float* __restrict__ w, __half* __restrict__ img, int n_out, int n_rows,
                                         int k_real, int k_groups, int k_map_c, int k_map_cp,
                                         const float* __restrict__ bias, int bias_col) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (kg, n)
  if (i >= k_groups * n_rows) return;
  int kg = i / n_rows, n = i - kg * n_rows;
  __half* dst = img + (size_t)i * 8;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    int k = kg * 8 + e;
    float v = 0.0f;
    if (n < n_out) {
      if (k_map_cp > 0) {
        int pair = k / k_map_cp, c = k - pair * k_map_cp;
        int col = pair * k_map_c + c;
        if (c < k_map_c && col < k_real) v = w[(size_t)n * k_real + col];
      } else if (k < k_real) {
        v = w[(size_t)n * k_real + k];
      } else if (k == bias_col && bias != nullptr) {
        v = bias[n];  // multiplied by the constant-1 input column
      }
    }
    dst[e] = __float2half_rn(v);
  }
}

// The same image with the K positions taken from a table: map[k] = column of w, -2 = bias, -1 = zero.
__global__ void pack_weight_image_mapped_kernel(const float* __restrict__ w, __half* __restrict__ img, int n_out, int n_rows,
                                                int k_real, int k_groups, const int* __restrict__ map,
                                                const float* __restrict__ bias) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (kg, n)
  if (i >= k_groups * n_rows) return;
  int kg = i / n_rows, n = i - kg * n_rows;
  __half* dst = img + (size_t)i * 8;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int col = map[kg * 8 + e];
    float v = 0.0f;
    if (n < n_out) {
      if (col >= 0 && col < k_real) v = w[(size_t)n * k_real + col];
      else if (col == -2 && bias != nullptr) v = bias[n];
    }
    dst[e] = __float2half_rn(v);
  }
}

template <int TA, int NSLOT, bool BASIS>
int launch_variant(const GnrModel* m, const TcArgs& args, cudaStream_t st) {
  const size_t smem = (size_t)WB_BYTES + W1_BYTES + W2_BYTES + W3_BYTES + (size_t)NSLOT * TA * A_BYTES +
                      (3 * HID + 2 * HID + 4) * sizeof(float) + 2 * NSLOT * sizeof(uint64_t) + 32;
  cudaError_t e = cudaFuncSetAttribute(mlp_tc_kernel<TA, NSLOT, BASIS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  mlp_tc_kernel<TA, NSLOT, BASIS><<<m->sm_count, NSLOT * 128, smem, st>>>(args);
  return (int)cudaGetLastError();
}

}  // namespace

int gnr_tc_basis_fused(const GnrModel* m) {
  // the operand buffer holds the products and one more k group (the view direction)
  return m->cfg.mlp_mode != 0 && m->mlp.n_prod % 16 == 0 && m->mlp.n_prod + 8 <= MAX_K0 && m->cfg.app_dim <= NB;
}

int gnr_tc_tile_bytes(const GnrModel* m) { return (m->mlp.n_prod / 8 + 1) * KG_BYTES; }

int gnr_mlp_tc_prepare(GnrModel* m, const float* basis_w, const float* w1, const float* w2, const float* w3, cudaStream_t st) {
  const GnrConfig& c = m->cfg;
  if (c.app_dim != APP || c.fea_pe != FPE || c.view_pe != VPE || c.hidden != HID) {
    gnr_set_error("tensor-core MLP supports app_dim 27, fea_pe 2, view_pe 2, featureC 128 (got %d, %d, %d, %d); use mlp_mode 0",
                  c.app_dim, c.fea_pe, c.view_pe, c.hidden);
    return -1;
  }
  if (m->mlp.tc_image) cudaFree(m->mlp.tc_image);
  m->mlp.tc_image = nullptr;
  // [basis][W1][W2][W3] and, for the fused appearance kernel, W1 once more with its K order permuted
  m->mlp.tc_image_bytes = (size_t)WB_BYTES + W1_BYTES + W2_BYTES + W3_BYTES + W1_BYTES + K1 * sizeof(int);
  GNR_CUDA_OK(cudaMalloc(&m->mlp.tc_image, m->mlp.tc_image_bytes));
  GNR_CUDA_OK(cudaMemsetAsync(m->mlp.tc_image, 0, m->mlp.tc_image_bytes, st));
  __half* img = reinterpret_cast<__half*>(m->mlp.tc_image);
  // the basis over PADDED channels (k = pair * cp + channel): what the fused paths multiply the products by, and, for a
  // channel slice of any width, what the slice projection does
  const int cp = (c.n_app + 15) / 16 * 16, kgb = c.n_pairs * cp / 8;
  if (c.app_dim <= NB && c.n_pairs * cp <= MAX_K0) {
    pack_weight_image_kernel<<<(kgb * NB + 255) / 256, 256, 0, st>>>(basis_w, img, c.app_dim, NB, c.n_pairs * c.n_app, kgb,
                                                                    c.n_app, cp, nullptr, -1);
  }
  // b1 / b2 in the m->mlp fp32 copies are zeros when the model has no biases
  pack_weight_image_kernel<<<(KG1 * HID + 255) / 256, 256, 0, st>>>(w1, img + WB_BYTES / 2, HID, HID, IN_DIM, KG1, 0, 0,
                                                                   m->mlp.b1, BIAS_COL1);
  pack_weight_image_kernel<<<(KG2 * HID + 255) / 256, 256, 0, st>>>(w2, img + (WB_BYTES + W1_BYTES) / 2, HID, HID, HID, KG2,
                                                                   0, 0, m->mlp.b2, BIAS_COL2);
  pack_weight_image_kernel<<<((HID / 8) * N3 + 255) / 256, 256, 0, st>>>(w3, img + (WB_BYTES + W1_BYTES + W2_BYTES) / 2, 3, N3,
                                                                        HID, HID / 8, 0, 0, nullptr, -1);
  {
    int map_h[K1];
    gnr_fused_k1_order(map_h);
    int* map_d = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(m->mlp.tc_image) + WB_BYTES + 2 * W1_BYTES + W2_BYTES + W3_BYTES);
    GNR_CUDA_OK(cudaMemcpyAsync(map_d, map_h, sizeof(map_h), cudaMemcpyHostToDevice, st));
    GNR_CUDA_OK(cudaStreamSynchronize(st));  // map_h is a stack array
    pack_weight_image_mapped_kernel<<<(KG1 * HID + 255) / 256, 256, 0, st>>>(
        w1, img + (WB_BYTES + W1_BYTES + W2_BYTES + W3_BYTES) / 2, HID, HID, IN_DIM, KG1, map_d, m->mlp.b1);
  }
  GNR_CUDA_OK(cudaGetLastError());
  return 0;
}

int launch_mlp_tc(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, int feat_stride, const float* feat_in,
                  float* feat_out, const unsigned char* prod_hi, const unsigned char* prod_lo, int tile_bytes, float* rgb,
                  int32_t* status, int force_unfused, cudaStream_t st, int basis_only) {
  if (!m->mlp.tc_image) {
    gnr_set_error("tensor-core MLP weights were not prepared");
    return -1;
  }
  if (feat_stride != FEAT_STRIDE) {
    gnr_set_error("tensor-core MLP expects a feature stride of %d floats", FEAT_STRIDE);
    return -1;
  }
  const bool fused = gnr_tc_basis_fused(m) != 0 && !force_unfused;
  TcArgs a;
  a.crd = c;
  a.feat_in = feat_in;
  a.feat_out = fused ? feat_out : nullptr;
  a.prod_hi = fused ? prod_hi : nullptr;
  a.prod_lo = fused ? prod_lo : nullptr;
  a.tile_bytes = tile_bytes;
  a.k0 = m->mlp.n_prod;
  a.w_image = (const unsigned char*)m->mlp.tc_image;
  a.w3 = m->mlp.w3;
  a.b1 = m->mlp.b1;
  a.b2 = m->mlp.b2;
  a.b3 = m->mlp.b3;
  a.rgb_out = rgb;
  a.status = status;
  a.kbits = p.kbits;
  a.basis_only = (basis_only && fused) ? 1 : 0;
  a.wait_limit = m->debug_wait_limit > 0 ? (uint32_t)m->debug_wait_limit : kWaitLimit;
  a.debug_skip_copy = m->debug_expire_wait;
  if (basis_only && !fused) {
    gnr_set_error("the projection-only launch needs the fused tensor-core path");
    return -1;
  }
  if (m->cfg.mlp_mode == 1) return fused ? launch_variant<2, 1, true>(m, a, st) : launch_variant<2, 1, false>(m, a, st);
  if (m->cfg.mlp_mode == 2) return fused ? launch_variant<1, 3, true>(m, a, st) : launch_variant<1, 3, false>(m, a, st);
  gnr_set_error("unknown mlp_mode %d", m->cfg.mlp_mode);
  return -1;
}
