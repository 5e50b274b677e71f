// Appearance gather + basis projection + MLP in ONE kernel, operands never leave the SM.
//
// compute_appfeature (app/models/gridnerf_sequential.py:829-871: per pair, bilinear plane sample x
// linear line sample, then basis_mat) followed by MLPRender_Fea.forward
// (app/models/mlp_render_fea.py:44-68).  The reference's own fused attempt keeps positional
// encoding and the GEMMs in one pass (dist_render/kernel/cuda_kernel/dal/pe_concate_mlp) behind a
// separate gather kernel; here the gather is in the same kernel too.
//
// One persistent CTA per SM, two groups of 128 threads; thread = appearance sample = row of a
// 128-row tile = lane of tensor memory.  Per tile a group
//   1. gathers: each thread interpolates the 144 plane x line products of its sample (packed fp16,
//      256-bit loads, the arithmetic of the stand-alone gather) and writes them with tcgen05.st into
//      tensor memory, where they ARE the A operand of the basis projection (72 columns of fp16 pairs);
//   2. F  = A0 * Wb^T                 tcgen05.mma, A from tensor memory, B (basis) from shared memory
//   3. A1 = [F, view, sin/cos ...]    registers -> tensor memory (80 columns)
//   4. D  = A1 * W1^T, A2 = relu(D), D = A2 * W2^T, A3 = relu(D), rgb = sigmoid(A3 * W3^T + b3)
//      every activation goes registers -> tensor memory -> MMA; biases ride in the MMAs.
// Shared memory holds only the four weight images (90 KB): no operand of a sample is ever written
// to shared or global memory, so the L1/shared-memory port carries the gather's loads and the
// weight fetches of the MMAs and nothing else, and the rest of the 256 KB array stays L1 cache for
// the texels.  While one group gathers (L1 port) the other group's MMAs run (tensor pipe).
//
// Tensor memory, 256 columns per group: R0 = [0, 128) accumulator D of layers 1 and 2;
// R1 = [128, 256): columns 0..79 the current A operand (A0, then A1, A2, A3: each is dead when the
// next is written), columns 96..127 the fp32 result of the basis projection and later of layer 3.
//
// Every wait on an mbarrier is bounded; when one expires the group raises
// status[GNR_ST_WAIT_EXPIRED] and stops taking tiles; before the CTA frees its tensor memory a
// group that stopped commits once more and waits (bounded) so that none of its MMAs is in flight.
#include <type_traits>

#include "gnr_gather.cuh"
#include "gnr_tc.cuh"

namespace {

constexpr int FG = 2;               // groups per CTA
constexpr int GROUP_COLS = 256;     // tensor-memory columns per group
constexpr int A_COL = HID;          // R1: A operand
constexpr int F_COL = HID + 96;     // R1: 32 fp32 columns (features, then the layer-3 result)
constexpr int PAIR_COLS = 24;       // 48 channels of a pair as fp16 pairs

struct FusedArgs {
  GnrCoords crd;
  const unsigned char* w_image;  // [basis][W1][W2][W3] fp16 operand images (gnr_mlp_tc_prepare)
  const float* b3;
  float* rgb_out;
  int32_t* status;
  int k0;                        // products per sample (n_pairs * 48)
  uint32_t wait_limit;           // iterations a bounded wait may take
  int debug_skip_commit;         // test hook: group 0 of CTA 0 leaves out the commit of its first basis GEMM
  long long* prof;               // null, or [FG][16] cycle sums per phase of the middle CTA (measurement aid)
};

template <int NP, bool PROF>
__global__ void __launch_bounds__(FG * 128, 1) app_mlp_fused_kernel(GnrSampleParams p, PlaneSet planes, FusedArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* s_wb = smem;
  unsigned char* s_w1 = s_wb + WB_BYTES;
  unsigned char* s_w2 = s_w1 + W1_BYTES;
  unsigned char* s_w3h = s_w2 + W2_BYTES;
  float* s_b3 = reinterpret_cast<float*>(s_w3h + W3_BYTES);
  uint64_t* s_mbar = reinterpret_cast<uint64_t*>(s_b3 + 4);  // [FG] MMA completion
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_mbar + FG);
  volatile uint32_t* s_flag = s_tmem + 1;                    // [FG] outcome of a group's last wait

  const int tid = threadIdx.x, warp = tid >> 5;
  const int warp_u = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int slot = warp_u >> 2, row = tid & 127;
  const int warp_in_group = warp_u & 3;  // GEMM i of a tile is issued by warp i of the group: the ~50-90 cycles an MMA
                                         // takes to issue are then spread over the four warps instead of adding up in one

  {
    const uint4* src = reinterpret_cast<const uint4*>(a.w_image);
    uint4* dst = reinterpret_cast<uint4*>(s_wb);
    for (int i = tid; i < (WB_BYTES + W1_BYTES + W2_BYTES + W3_BYTES) / 16; i += FG * 128) dst[i] = src[i];
    if (tid < 4) s_b3[tid] = a.b3[tid];
    if (tid == 0) {
      for (int s = 0; s < FG; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_mbar[s])));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                   "r"((uint32_t)(FG * GROUP_COLS)));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *s_tmem, 0);
  const uint32_t d_tmem = tmem_base + (uint32_t)(slot * GROUP_COLS);  // R0
  const uint32_t a_tmem = d_tmem + A_COL;                             // R1, A operand
  const uint32_t f_tmem = d_tmem + F_COL;                             // R1, fp32 result columns
  const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
  const uint32_t wb_addr = smem_u32(s_wb), w1_addr = smem_u32(s_w1), w2_addr = smem_u32(s_w2), w3_addr = smem_u32(s_w3h);
  const uint32_t mbar = smem_u32(&s_mbar[slot]);
  const int bar_id = 1 + slot;
  s_flag += slot;
  uint32_t parity = 0;
  bool expired = false;

  const long long total = min(a.crd.total_ptr ? (long long)*a.crd.total_ptr : a.crd.total_direct, a.crd.capacity);
  const long long n_tiles = (total + ROWS - 1) / ROWS;
  // a contiguous share of the list per CTA (neighbouring tiles are neighbouring rays: their texels
  // are still in this SM's L1), the two groups taking alternate tiles of it
  const long long per = (n_tiles + gridDim.x - 1) / gridDim.x;
  const long long t_beg = min(n_tiles, (long long)blockIdx.x * per), t_end = min(n_tiles, t_beg + per);
  const int ksteps0 = a.k0 >> 4;

#define GROUP_SYNC() asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory")
#define WAIT_OR_STOP()                                                   \
  if (!group_wait(mbar, parity, bar_id, row, s_flag, a.wait_limit)) {    \
    if (row == 0) atomicExch(a.status + GNR_ST_WAIT_EXPIRED, 1);         \
    expired = true;                                                      \
    break;                                                               \
  }                                                                      \
  parity ^= 1

  // ---- software pipeline: the products of a group's NEXT tile are gathered into registers (72 packed fp16
  // pairs per thread) in the shadows of the current tile's MMAs: positions and L1 prefetches behind the
  // projection, one plane/line pair behind each of the three layers, so the L1 port works while the tensor
  // pipe does and a tile starts with its A0 ready
  uint32_t nq[3 * PAIR_COLS];
  float nx = 0.0f, ny = 0.0f, nz = 0.0f, nview[3] = {0.0f, 0.0f, 0.0f};
  auto fetch_pos = [&](long long t) {
    const long long jr = t * ROWS + row;
    // rows past the end repeat the last entry (no divergence around the warp-wide tensor-memory
    // instructions) and write nothing
    sample_xyz(p, a.crd, jr < total ? jr : total - 1, nx, ny, nz, nview);
  };
  auto gather_pair = [&](auto pair_c) {
    constexpr int pi = decltype(pair_c)::value;
    if (pi >= planes.n) {  // fewer than three pairs: the columns stay zero
#pragma unroll
      for (int e = 0; e < PAIR_COLS; ++e) nq[pi * PAIR_COLS + e] = 0u;
      return;
    }
    const GnrPlane& pl = planes.p[pi];
    PairTapsH2 t;
    if (NP == 3) {
      const Tap tx = make_tap(nx, planes.p[0].fw, planes.p[0].W);
      const Tap ty = make_tap(ny, planes.p[0].fh, planes.p[0].H);
      const Tap tz = make_tap(nz, planes.p[0].fl, planes.p[0].L);
      t = pi == 0 ? make_pair_taps_h2(pl, tx, ty, tz) : (pi == 1 ? make_pair_taps_h2(pl, tx, tz, ty) : make_pair_taps_h2(pl, ty, tz, tx));
    } else {
      const float u = pick(nx, ny, nz, pl.mat0), v = pick(nx, ny, nz, pl.mat1), l = pick(nx, ny, nz, pl.vec);
      t = make_pair_taps_h2(pl, make_tap(u, pl.fw, pl.W), make_tap(v, pl.fh, pl.H), make_tap(l, pl.fl, pl.L));
    }
#pragma unroll
    for (int g = 0; g < 3; ++g) {
      uint32_t q[8];
      pair_round_h2(pl, t, g, q);
#pragma unroll
      for (int e = 0; e < 8; ++e) nq[pi * PAIR_COLS + g * 8 + e] = q[e];
    }
  };
  // Brings the lines of the next tile's texels into L1 well before the gather reads them: per pair the
  // two upper corners, the two lower corners and the two line entries are 192 contiguous bytes each.
  auto prefetch_next = [&]() {
#pragma unroll
    for (int pi = 0; pi < 3; ++pi) {
      if (pi < planes.n) {
        const GnrPlane& pl = planes.p[pi];
        const float u = pick(nx, ny, nz, pl.mat0), v = pick(nx, ny, nz, pl.mat1), l = pick(nx, ny, nz, pl.vec);
        const Tap tu = make_tap(u, pl.fw, pl.W), tv = make_tap(v, pl.fh, pl.H), tl = make_tap(l, pl.fl, pl.L);
        const uint32_t nw = (uint32_t)tv.i0 * (uint32_t)pl.W + (uint32_t)tu.i0;
        const unsigned char* r0 = reinterpret_cast<const unsigned char*>(pl.plane) + (size_t)nw * 96u;
        const unsigned char* r1 = r0 + (size_t)pl.W * 96u;
        const unsigned char* r2 = reinterpret_cast<const unsigned char*>(pl.line) + (size_t)tl.i0 * 96u;
        const unsigned char* rs[3] = {r0, r1, r2};
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          asm volatile("prefetch.global.L1 [%0];" ::"l"(rs[k]));
          asm volatile("prefetch.global.L1 [%0];" ::"l"(rs[k] + 128));
          asm volatile("prefetch.global.L1 [%0];" ::"l"(rs[k] + 191));
        }
      }
    }
  };
  using P0 = std::integral_constant<int, 0>;
  using P1 = std::integral_constant<int, 1>;
  using P2 = std::integral_constant<int, 2>;
  if (t_beg + slot < t_end) {
    fetch_pos(t_beg + slot);
    gather_pair(P0{});
    gather_pair(P1{});
    gather_pair(P2{});
  }

  // phase timer of one thread per group of one CTA (only when a buffer was passed)
  const bool prof_on = PROF && a.prof != nullptr && row == 0 && blockIdx.x == gridDim.x / 2;
  long long pacc[16], plast = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) pacc[i] = 0;
#define PROF_MARK(k)               \
  if (PROF && prof_on) {           \
    const long long now = clock64(); \
    pacc[k] += now - plast;        \
    plast = now;                   \
  }
  if (PROF && prof_on) plast = clock64();

  for (long long tile = t_beg + slot; tile < t_end; tile += FG) {
    const long long j = tile * ROWS + row;
    const bool live = j < total;
    const bool has_next = tile + FG < t_end;  // (the same for every thread of the group)
    // ---- this tile's products: registers -> tensor memory ------------------------------------------------
    const float view[3] = {nview[0], nview[1], nview[2]};
    tmem_st32(a_tmem + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&nq[0]));
    tmem_st32(a_tmem + lane_off + 32, *reinterpret_cast<uint32_t(*)[32]>(&nq[32]));
    tmem_st8(a_tmem + lane_off + 64, *reinterpret_cast<uint32_t(*)[8]>(&nq[64]));
    tmem_st_wait();
    tc_fence_before();
    GROUP_SYNC();
    PROF_MARK(0);

    // ---- F = A0 * Wb^T ---------------------------------------------------------------------------------
    if (warp_in_group == 0) {
      tc_fence_after();
      const uint32_t leader = elect_one();
#pragma unroll
      for (int ks = 0; ks < MAX_K0 / 16; ++ks) {
        if (ks < ksteps0)
          mma_f16_ts(f_tmem, a_tmem + ks * 8, make_desc(wb_addr + ks * 2 * KGB_BYTES, KGB_BYTES), kIdescBasis, ks > 0 ? 1u : 0u, leader);
      }
      const bool skip = a.debug_skip_commit != 0 && blockIdx.x == 0 && slot == 0 && tile == t_beg;
      mma_commit(mbar, skip ? 0u : leader);
      __syncwarp();
    }
    PROF_MARK(1);
    if (has_next) {  // behind the projection: the next tile's positions, and its texels on their way into L1
      fetch_pos(tile + FG);
      prefetch_next();
    }
    PROF_MARK(2);
    WAIT_OR_STOP();
    PROF_MARK(3);
    float f[32];
    {
      uint32_t v[32];
      tmem_ld32(f_tmem + lane_off, v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
    }

    // ---- A1: features, view direction and their positional encodings ----------------------------------------
    {
      float x[K1];
#pragma unroll
      for (int i = 0; i < APP; ++i) x[i] = f[i];
#pragma unroll
      for (int i = 0; i < 3; ++i) x[APP + i] = view[i];
#pragma unroll
      for (int i = 0; i < APP; ++i) {  // sin/cos of v and 2 v: one sincos, then the double-angle identities
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
      uint32_t h[K1 / 2];
#pragma unroll
      for (int i = 0; i < K1 / 2; ++i) h[i] = pack_h2(x[2 * i], x[2 * i + 1]);
      tmem_st32(a_tmem + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&h[0]));
      tmem_st32(a_tmem + lane_off + 32, *reinterpret_cast<uint32_t(*)[32]>(&h[32]));
      tmem_st16(a_tmem + lane_off + 64, *reinterpret_cast<uint32_t(*)[16]>(&h[64]));
    }
    tmem_st_wait();
    tc_fence_before();
    GROUP_SYNC();
    PROF_MARK(4);

    // ---- D = A1 * W1^T ---------------------------------------------------------------------------------------
    if (warp_in_group == 1) {
      tc_fence_after();
      const uint32_t leader = elect_one();
#pragma unroll
      for (int ks = 0; ks < K1 / 16; ++ks)
        mma_f16_ts(d_tmem, a_tmem + ks * 8, make_desc(w1_addr + ks * 2 * KG_BYTES, KG_BYTES), kIdescHid, ks > 0 ? 1u : 0u, leader);
      mma_commit(mbar, leader);
      __syncwarp();
    }
    PROF_MARK(5);
    if (has_next) gather_pair(P0{});  // behind layer 1
    PROF_MARK(6);
    WAIT_OR_STOP();
    PROF_MARK(7);

    // ---- A2 = relu(D) (D already holds b1), the constant-1 column of b2, padding ------------------------------
#pragma unroll
    for (int cb = 0; cb < HID / 64; ++cb) {
      uint32_t v[64];
      tmem_ld32(d_tmem + lane_off + cb * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
      tmem_ld32(d_tmem + lane_off + cb * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
      tmem_ld_wait();
      uint32_t h[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) h[e] = pack_h2_relu(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
      tmem_st32(a_tmem + lane_off + cb * 32, h);
    }
    {
      const uint32_t tail[8] = {pack_h2(1.0f, 0.0f), 0u, 0u, 0u, 0u, 0u, 0u, 0u};  // k = 128 is the bias input, 129..143 padding
      tmem_st8(a_tmem + lane_off + HID / 2, tail);
    }
    tmem_st_wait();
    tc_fence_before();
    GROUP_SYNC();
    PROF_MARK(8);

    // ---- D = A2 * W2^T ---------------------------------------------------------------------------------------
    if (warp_in_group == 2) {
      tc_fence_after();
      const uint32_t leader = elect_one();
#pragma unroll
      for (int ks = 0; ks < K2 / 16; ++ks)
        mma_f16_ts(d_tmem, a_tmem + ks * 8, make_desc(w2_addr + ks * 2 * KG_BYTES, KG_BYTES), kIdescHid, ks > 0 ? 1u : 0u, leader);
      mma_commit(mbar, leader);
      __syncwarp();
    }
    PROF_MARK(9);
    if (has_next) gather_pair(P1{});  // behind layer 2
    PROF_MARK(10);
    WAIT_OR_STOP();
    PROF_MARK(11);

    // ---- A3 = relu(D), rgb = sigmoid(A3 * W3^T + b3) ---------------------------------------------------------
#pragma unroll
    for (int cb = 0; cb < HID / 64; ++cb) {
      uint32_t v[64];
      tmem_ld32(d_tmem + lane_off + cb * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
      tmem_ld32(d_tmem + lane_off + cb * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
      tmem_ld_wait();
      uint32_t h[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) h[e] = pack_h2_relu(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
      tmem_st32(a_tmem + lane_off + cb * 32, h);
    }
    tmem_st_wait();
    tc_fence_before();
    GROUP_SYNC();
    PROF_MARK(12);
    if (warp_in_group == 3) {
      tc_fence_after();
      const uint32_t leader = elect_one();
#pragma unroll
      for (int ks = 0; ks < HID / 16; ++ks)
        mma_f16_ts(f_tmem, a_tmem + ks * 8, make_desc(w3_addr + ks * 2 * KG3_BYTES, KG3_BYTES), kIdescOut, ks > 0 ? 1u : 0u, leader);
      mma_commit(mbar, leader);
      __syncwarp();
    }
    if (has_next) gather_pair(P2{});  // behind layer 3
    WAIT_OR_STOP();
    PROF_MARK(13);
    {
      uint32_t r[4];
      tmem_ld4(f_tmem + lane_off, r);
      tmem_ld_wait();
      if (live) {
        float* out = a.rgb_out + (size_t)j * 3;
        out[0] = 1.0f / (1.0f + expf(-(s_b3[0] + __uint_as_float(r[0]))));
        out[1] = 1.0f / (1.0f + expf(-(s_b3[1] + __uint_as_float(r[1]))));
        out[2] = 1.0f / (1.0f + expf(-(s_b3[2] + __uint_as_float(r[2]))));
      }
    }
    tc_fence_before();  // this tile's tensor-memory reads come before the next tile's writes
    PROF_MARK(14);
  }
#undef WAIT_OR_STOP
#undef PROF_MARK
  if (PROF && prof_on) {
#pragma unroll
    for (int i = 0; i < 16; ++i) a.prof[slot * 16 + i] = pacc[i];
  }

  // ---- teardown ---------------------------------------------------------------------------------------------
  if (expired) {
    // MMAs of this group may still be running: commit once more and wait for them, so that nothing
    // writes tensor memory after it has been freed
    if (warp_in_group == 0) {
      const uint32_t leader = elect_one();
      mma_commit(mbar, leader);
      __syncwarp();
    }
    group_wait(mbar, parity, bar_id, row, s_flag, a.wait_limit);
  }
#undef GROUP_SYNC
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(FG * GROUP_COLS)));
  }
}

constexpr size_t kFusedSmem = (size_t)WB_BYTES + W1_BYTES + W2_BYTES + W3_BYTES + 4 * sizeof(float) + FG * sizeof(uint64_t) + 64;

}  // namespace

int gnr_app_fusable(const GnrModel* m) {
  // fp16 appearance planes of 48 (padded) channels, the single-fp16 tensor-core mode, and a product count
  // that fits the 80 operand columns
  return m->cfg.mlp_mode == 2 && m->cfg.app_storage == 1 && m->cfg.unfused_appearance == 0 && gnr_tc_basis_fused(m) &&
         m->app[0].C == 48 && m->mlp.n_prod == m->cfg.n_pairs * 48 && m->mlp.n_prod <= MAX_K0;
}

int launch_app_mlp_fused(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, float* rgb, int32_t* status,
                         cudaStream_t st) {
  if (!m->mlp.tc_image) {
    gnr_set_error("tensor-core MLP weights were not prepared");
    return -1;
  }
  PlaneSet set = make_set(m->app, m->cfg.n_pairs);
  FusedArgs a;
  a.crd = c;
  a.w_image = (const unsigned char*)m->mlp.tc_image;
  a.b3 = m->mlp.b3;
  a.rgb_out = rgb;
  a.status = status;
  a.k0 = m->mlp.n_prod;
  a.wait_limit = m->debug_wait_limit > 0 ? (uint32_t)m->debug_wait_limit : kWaitLimit;
  a.debug_skip_commit = m->debug_expire_wait;
  a.prof = m->debug_prof;
  auto launch = [&](auto kernel) -> int {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFusedSmem);
    if (e != cudaSuccess) return (int)e;
    kernel<<<m->sm_count, FG * 128, kFusedSmem, st>>>(p, set, a);
    return 0;
  };
  int rc;
  if (a.prof) rc = standard_vm3(set) ? launch(app_mlp_fused_kernel<3, true>) : launch(app_mlp_fused_kernel<0, true>);
  else rc = standard_vm3(set) ? launch(app_mlp_fused_kernel<3, false>) : launch(app_mlp_fused_kernel<0, false>);
  if (rc) return rc;
  return (int)cudaGetLastError();
}
