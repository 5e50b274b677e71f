// Appearance gather + basis projection + MLP in ONE kernel, operands never leave the SM.
//
// compute_appfeature (app/models/gridnerf_sequential.py:829-871: per pair, bilinear plane sample x
// linear line sample, then basis_mat) followed by MLPRender_Fea.forward
// (app/models/mlp_render_fea.py:44-68).  The reference's own fused attempt keeps positional
// encoding and the GEMMs in one pass (dist_render/kernel/cuda_kernel/dal/pe_concate_mlp) behind a
// separate gather kernel; here the gather is in the same kernel too.
//
// One persistent CTA per SM, three groups of 256 threads (768 threads, 80 registers each); a group works on
// one 128-sample tile at a time.  Row r of the tile (= lane r of tensor memory) belongs to TWO threads of the
// group, one in each half of it (warps 0-3 and 4-7; warp w of either half owns lanes 32 (w % 4) ..): every
// per-row phase is split between them by columns, so each phase takes half as long and the SM holds 24 warps
// whose loads hide each other's latency.  Per tile a group
//   1. gathers: the 144 plane x line products of a sample as nine rounds of 16 channels (packed fp16,
//      256-bit loads, the arithmetic of the stand-alone gather); half 0 takes rounds 0-4, half 1
//      rounds 5-8, and each round goes with one tcgen05.st straight into tensor memory, where the
//      products ARE the A operand of the basis projection;
//   2. F  = A0 * Wb^T                 tcgen05.mma, A from tensor memory, B (basis) from shared memory
//   3. A1 = [F, view, sin/cos ...]    registers -> tensor memory: half 0 encodes features 0-13, half 1
//                                     features 14-26 and the view direction, 40 columns each (the K
//                                     order of layer 1 is permuted to make the halves contiguous;
//                                     the W1 image carries the same permutation)
//   4. D  = A1 * W1^T, A2 = relu(D), D = A2 * W2^T, A3 = relu(D), rgb = sigmoid(A3 * W3^T + b3)
//      every activation goes registers -> tensor memory -> MMA (half h converts columns 64 h .. of D);
//      biases ride in the MMAs.
// Shared memory holds only the four weight images (90 KB): no operand of a sample is ever written
// to shared or global memory, so the L1/shared-memory port carries the gather's loads and the
// weight fetches of the MMAs and nothing else, and the rest of the 256 KB array stays L1 cache for
// the texels.  While one group gathers (L1 port) the other groups' MMAs run (tensor pipe).  GEMM i of
// a tile is issued by warp i of the group, so the issue time of the MMAs is spread over four warps.
// The (ray, sample) of a row is fetched two tiles ahead and the ray itself one tile ahead, so the
// dependent loads behind a list entry are never waited for.
//
// Tensor memory (512 columns): a tile needs an 80-column operand buffer for its whole life (A0, then A1,
// A2, A3: each is dead when the next is written) but its 128-column fp32 accumulator only from the
// projection on, about 60 % of it.  So the three groups own the operand buffers [80 g, 80 g + 80) and SHARE
// two accumulators, [256, 384) and [384, 512): the n-th tile of the CTA (group n % 3) accumulates in D[n & 1]
// and takes it over from tile n - 2, whose group counts a release in shared memory as soon as that tile's
// last result is in registers; the warp that issues a tile's first MMA waits (bounded) for that count.  The
// 32 fp32 columns of the projection, and later the layer-3 result, sit at the start of the same accumulator.
// With two groups (GnrConfig.unfused_appearance = 3) tile n - 2 is the group's own previous tile and nothing
// is waited for; three tiles in flight measured 14.4 against 17.5 ms per city frame.
//
// LAT variant (gnr_build_appearance_lattice): the 27 projected features are themselves trilinear in the
// position (sum over pairs and channels of basis weight x plane texel x line entry at the eight surrounding
// grid points), so they can be baked into one lattice of 32 fp16 channels per grid point; a sample then
// reads 8 x 64 bytes instead of 18 x 96, and steps 1 and 2 disappear (the tile starts at step 3).
//
// Every wait on an mbarrier is bounded; when one expires the group raises
// status[GNR_ST_WAIT_EXPIRED] and stops taking tiles; before the CTA frees its tensor memory a
// group that stopped commits once more and waits (bounded) so that none of its MMAs is in flight.
#include <type_traits>

#include "gnr_gather.cuh"
#include "gnr_tc.cuh"

namespace {

constexpr int MAX_FG = 3;           // groups per CTA: 3 (default) or 2
constexpr int GT = 256;             // threads per group (two per row)
constexpr int TMEM_COLS = 512;      // the whole tensor memory of the SM
constexpr int A_COLS = 80;          // operand columns of a group, at [80 g, 80 g + 80)
constexpr int D_COL = 256;          // the two accumulators: [256, 384) and [384, 512)

struct FusedArgs {
  const float* rays;             // [n][6]
  const float* t_min;            // [n]
  const uint32_t* ids;           // appearance list: ray << kbits | sample
  const int32_t* total_ptr;      // length of the list (device), or null ...
  long long total_direct;        // ... then this host count (point mode)
  long long capacity;
  const float* xyz_direct;       // point mode: [n][3] normalised positions
  const float* view_direct;      // point mode: [n][3] view directions
  int point_stride;              // floats between the rows of consecutive points in either array
  const unsigned char* w_image;  // [basis][W1][W2][W3][W1 with permuted K] fp16 operand images
  const float* b3;
  float* rgb_out;
  int32_t* status;
  int k0;                        // products per sample (n_pairs * 48)
  uint32_t wait_limit;           // iterations a bounded wait may take
  int debug_skip_commit;         // test hook: group 0 of CTA 0 leaves out the commit of its first basis GEMM
  long long* prof;               // null, or [groups][16] cycle sums per phase of the middle CTA (measurement aid)
  const unsigned char* lat;      // LAT: projected-feature lattice [gx][gy][gz][32] fp16 (gnr_build_appearance_lattice)
  int lat_g[3];                  // its grid
  const float* feat;             // SRC 2: [n][feat_stride] fp32 projected features of the points
  int feat_stride;
  const unsigned char* parts;    // SRC 3: n_parts buffers of fp16 rows of 32 (64 bytes), part w starting part_stride rows in
  int n_parts;
  long long part_stride;
  int blk_px, blk_bx, blk_by;    // list mode at a block owner (blk_px > 0): positions, computed in the sampler's global
  float blk_pw, blk_ph;          // box, are then expressed in the coordinates of block (blk_bx, blk_by)
};

struct RaySample {  // what a row needs of its list entry
  float o[3], d[3], t_min;
  int k;
};

// SRC: where a tile's 27 projected features come from: 0 = gathered from the planes and lines and projected
// here, 1 = the projected-feature lattice, 2 = given per point (features computed elsewhere, e.g. summed over
// the channel slices of a tensor-parallel group), 3 = given per point as n_parts partial rows of 32 fp16 (the rows a
// tensor-parallel rank received from its peers), summed here in fp32; 1, 2 and 3 start a tile at step 3.
template <int NP, bool PROF, bool POINTS, int SRC, int FG>
__global__ void __launch_bounds__(FG * GT, 1) app_mlp_fused_kernel(GnrSampleParams p, PlaneSet planes, FusedArgs a) {
  constexpr bool LAT = SRC == 1, FEAT = SRC == 2, PARTS = SRC == 3;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* s_wb = smem;
  unsigned char* s_w1 = s_wb + WB_BYTES;  // layer 1, K permuted (see the header of this file)
  unsigned char* s_w2 = s_w1 + W1_BYTES;
  unsigned char* s_w3h = s_w2 + W2_BYTES;
  float* s_b3 = reinterpret_cast<float*>(s_w3h + W3_BYTES);
  uint64_t* s_mbar = reinterpret_cast<uint64_t*>(s_b3 + 4);  // [FG] MMA completion
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_mbar + FG);
  volatile uint32_t* s_flag = s_tmem + 1;                    // [FG] outcome of a group's last wait
  uint32_t* s_rel = s_tmem + 1 + MAX_FG;                     // [2] releases of each accumulator so far (4 per tile)

  const int tid = threadIdx.x, warp = tid >> 5;
  const int warp_u = __shfl_sync(0xffffffffu, tid >> 5, 0);  // the same number, known to be warp-uniform
  const int slot = warp_u >> 3;                              // group
  const int wg = warp_u & 7;                                 // warp in group
  const int half = wg >> 2;                                  // which half of every row's columns this thread takes
  const int row = tid & 127;
  const int tg = tid & (GT - 1);                             // thread in group

  {
    // weights -> shared memory: basis, W1 (the permuted image, stored last in global memory), W2, W3
    const uint4* src = reinterpret_cast<const uint4*>(a.w_image);
    const uint4* src_w1p = reinterpret_cast<const uint4*>(a.w_image + WB_BYTES + W1_BYTES + W2_BYTES + W3_BYTES);
    uint4* dst = reinterpret_cast<uint4*>(s_wb);
    constexpr int kAll = (WB_BYTES + W1_BYTES + W2_BYTES + W3_BYTES) / 16, kW1Beg = WB_BYTES / 16, kW1End = (WB_BYTES + W1_BYTES) / 16;
    for (int i = tid; i < kAll; i += FG * GT) dst[i] = (i >= kW1Beg && i < kW1End) ? src_w1p[i - kW1Beg] : src[i];
    if (tid < 4) s_b3[tid] = a.b3[tid];
    if (tid == 0) {
      for (int s = 0; s < FG; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_mbar[s])));
      s_rel[0] = 0u;
      s_rel[1] = 0u;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                   "r"((uint32_t)TMEM_COLS));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *s_tmem, 0);
  const uint32_t a_tmem = tmem_base + (uint32_t)(slot * A_COLS);      // this group's A operand
  const uint32_t rel0 = smem_u32(&s_rel[0]);
  const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;        // the lane quarter this warp may touch
  const uint32_t wb_addr = smem_u32(s_wb), w1_addr = smem_u32(s_w1), w2_addr = smem_u32(s_w2), w3_addr = smem_u32(s_w3h);
  const uint32_t mbar = smem_u32(&s_mbar[slot]);
  const int bar_id = 1 + slot;
  s_flag += slot;
  uint32_t parity = 0;
  bool expired = false;

  const long long total = min(a.total_ptr ? (long long)*a.total_ptr : a.total_direct, a.capacity);
  const long long n_tiles = (total + ROWS - 1) / ROWS;
  // a contiguous share of the list per CTA (neighbouring tiles are neighbouring rays: their texels
  // are still in this SM's L1), the two groups taking alternate tiles of it
  const long long per = (n_tiles + gridDim.x - 1) / gridDim.x;
  const long long t_beg = min(n_tiles, (long long)blockIdx.x * per), t_end = min(n_tiles, t_beg + per);
  const int ksteps0 = a.k0 >> 4;
  const uint32_t kmask = (1u << p.kbits) - 1u;

#define GROUP_SYNC() asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory")
#define WAIT_OR_STOP()                                                          \
  if (!group_wait(mbar, parity, bar_id, tg, s_flag, a.wait_limit, GT)) {        \
    if (tg == 0) atomicExch(a.status + GNR_ST_WAIT_EXPIRED, 1);                 \
    expired = true;                                                             \
    break;                                                                      \
  }                                                                             \
  parity ^= 1
  // phase timer of one thread per group of one CTA (only when a buffer was passed)
  const bool prof_on = PROF && a.prof != nullptr && tg == 0 && blockIdx.x == gridDim.x / 2;
  long long pacc[16], plast = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) pacc[i] = 0;
#define PROF_MARK(k)                 \
  if (PROF && prof_on) {             \
    const long long now = clock64(); \
    pacc[k] += now - plast;          \
    plast = now;                     \
  }

  // ---- list entry -> ray, two tiles ahead; ray -> registers, one tile ahead ----------------------------------
  // rows past the end of the list repeat its last entry (no divergence around the warp-wide tensor-memory
  // instructions) and write nothing
  auto entry_of = [&](long long t) -> uint32_t {
    const long long jr = t * ROWS + row;
    const long long at = jr < total ? jr : total - 1;
    if (POINTS) return (uint32_t)at;  // point mode: the "entry" is the point's own number
    return __ldg(a.ids + at);
  };
  auto load_ray = [&](uint32_t id) -> RaySample {
    RaySample r;
    if (POINTS) {  // o = the normalised position itself, d = the view direction
      const float* px = a.xyz_direct + (size_t)id * a.point_stride;
      const float* pv = a.view_direct + (size_t)id * a.point_stride;
      r.o[0] = __ldg(px + 0);
      r.o[1] = __ldg(px + 1);
      r.o[2] = __ldg(px + 2);
      r.d[0] = __ldg(pv + 0);
      r.d[1] = __ldg(pv + 1);
      r.d[2] = __ldg(pv + 2);
      r.t_min = 0.0f;
      r.k = 0;
      return r;
    }
    const uint32_t ray = id >> p.kbits;
    const float* src = a.rays + (size_t)ray * 6;
    r.o[0] = __ldg(src + 0);
    r.o[1] = __ldg(src + 1);
    r.o[2] = __ldg(src + 2);
    r.d[0] = __ldg(src + 3);
    r.d[1] = __ldg(src + 4);
    r.d[2] = __ldg(src + 5);
    r.t_min = __ldg(a.t_min + ray);
    r.k = (int)(id & kmask);
    return r;
  };
  uint32_t id_ahead = 0;  // entry of this group's tile after the next
  RaySample next_ray = {};
  if (t_beg + slot < t_end) {
    next_ray = load_ray(entry_of(t_beg + slot));
    if (t_beg + slot + FG < t_end) id_ahead = entry_of(t_beg + slot + FG);
  }
  if (PROF && prof_on) plast = clock64();

  for (long long tile = t_beg + slot; tile < t_end; tile += FG) {
    const long long j = tile * ROWS + row;
    const bool live = j < total;
    // The n-th tile of this CTA (counted over all groups) accumulates in D[n & 1]: its own group's for two
    // groups; with three groups the accumulator of the tile two before it, which that tile's group hands on
    // when it has read its last result.  f_tmem: the 32 fp32 columns of the projection and, later, of layer 3,
    // at the start of the same accumulator (each is read before the next MMA that writes there is issued).
    const uint32_t n_cta = (uint32_t)(tile - t_beg);
    const uint32_t d_tmem = tmem_base + (uint32_t)D_COL + (n_cta & 1u) * (uint32_t)HID;
    const uint32_t f_tmem = d_tmem;
    // Releases are COUNTED (one per warp that read the tile's last result, four per tile), not phases of an
    // mbarrier: a group meets an accumulator only every other tile of its own, so it would skip phases, and a
    // phase bit cannot tell "not yet" from "twice since".
    const uint32_t rel = rel0 + (n_cta & 1u) * 4u;
    auto acquire_d = [&]() -> bool {  // by every lane of the warp that issues the tile's first MMA
      if (FG == 2 || n_cta < 2u) return true;
      const uint32_t want = 4u * (n_cta >> 1);  // every earlier tile on this accumulator has been read out
      bool ok = false;
      for (uint32_t it = 0; it < a.wait_limit; ++it) {
        uint32_t seen;
        asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(seen) : "r"(rel) : "memory");
        if (seen >= want) {
          ok = true;
          break;
        }
        if (it > 64) __nanosleep(64);
      }
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      return ok;
    };
    const RaySample cur = next_ray;
    if (tile + FG < t_end) next_ray = load_ray(id_ahead);              // (not needed before the next iteration)
    if (tile + 2 * FG < t_end) id_ahead = entry_of(tile + 2 * FG);

    uint32_t v[32];  // the 27 projected features of this row as fp32 bits (half 0 reads v[0..13], half 1 v[14..26])
    if constexpr (PARTS) {
      // ---- features as the fp32 sum of n_parts fp16 rows (part w of row r at (w * part_stride + r) * 64 bytes): this
      // half's columns, parts added in order -----------------------------------------------------------------------
      const size_t r = (size_t)(j < total ? j : total - 1);
      float acc[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) acc[e] = 0.0f;
      for (int w = 0; w < a.n_parts; ++w) {
        // half 0: columns 0..15 (uses 0..13); half 1: columns 8..31 are loaded, 14..26 used -> acc[e] = column 14 + e
        const uint4* src = reinterpret_cast<const uint4*>(a.parts + ((size_t)w * a.part_stride + r) * 64);
        if (half == 0) {
          const uint4 c0 = __ldg(src), c1 = __ldg(src + 1);
          const uint32_t u[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
          for (int e = 0; e < 7; ++e) {
            const float2 f = __half22float2(as_h2(u[e]));
            acc[2 * e] += f.x;
            acc[2 * e + 1] += f.y;
          }
        } else {
          const uint4 c1 = __ldg(src + 1), c2 = __ldg(src + 2), c3 = __ldg(src + 3);
          const uint32_t u[12] = {c1.x, c1.y, c1.z, c1.w, c2.x, c2.y, c2.z, c2.w, c3.x, c3.y, c3.z, c3.w};  // columns 8..31
#pragma unroll
          for (int e = 0; e < 13; ++e) {  // column 14 + e = element (6 + e) of the 24 loaded
            const float2 f = __half22float2(as_h2(u[(6 + e) >> 1]));
            acc[e] += ((6 + e) & 1) ? f.y : f.x;
          }
        }
      }
      if (half == 0) {
#pragma unroll
        for (int e = 0; e < 14; ++e) v[e] = __float_as_uint(acc[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 13; ++e) v[14 + e] = __float_as_uint(acc[e]);
      }
      PROF_MARK(0);
    } else if constexpr (FEAT) {
      // ---- features given per point: this half's 14 / 13 values of the row --------------------------------------
      const float* src = a.feat + (size_t)(j < total ? j : total - 1) * a.feat_stride + (half ? 14 : 0);
      if (half == 0) {
#pragma unroll
        for (int e = 0; e < 14; ++e) v[e] = __float_as_uint(__ldg(src + e));
      } else {
#pragma unroll
        for (int e = 0; e < 13; ++e) v[14 + e] = __float_as_uint(__ldg(src + e));
      }
      PROF_MARK(0);
    } else if constexpr (LAT) {
      // ---- features straight from the projected-feature lattice: trilinear interpolation of this half's 16
      // channels (8 taps x 32 bytes, fp32 accumulation); no products, no projection GEMM -------------------
      const float t = POINTS ? 0.0f : gnr_sample_t(p, cur.t_min, cur.k);
      float x = POINTS ? cur.o[0] : gnr_normalize(gnr_point(cur.o[0], cur.d[0], t), p.lo[0], p.inv[0]);
      float y = POINTS ? cur.o[1] : gnr_normalize(gnr_point(cur.o[1], cur.d[1], t), p.lo[1], p.inv[1]);
      const float z = POINTS ? cur.o[2] : gnr_normalize(gnr_point(cur.o[2], cur.d[2], t), p.lo[2], p.inv[2]);
      if (!POINTS && a.blk_px > 0) block_local((float)a.blk_bx, (float)a.blk_by, a.blk_pw, a.blk_ph, x, y, x, y);
      const Tap tx = make_tap(x, (float)(a.lat_g[0] - 1), a.lat_g[0]);
      const Tap ty = make_tap(y, (float)(a.lat_g[1] - 1), a.lat_g[1]);
      const Tap tz = make_tap(z, (float)(a.lat_g[2] - 1), a.lat_g[2]);
      const size_t gz = (size_t)a.lat_g[2], gyz = (size_t)a.lat_g[1] * gz;
      const size_t p000 = ((size_t)tx.i0 * (size_t)a.lat_g[1] + (size_t)ty.i0) * gz + (size_t)tz.i0;
      const unsigned char* base = a.lat + half * 32;
      const float wx[2] = {1.0f - tx.f1, tx.f1}, wy[2] = {1.0f - ty.f1, ty.f1}, wz[2] = {1.0f - tz.f1, tz.f1};
      H16 tap[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const size_t pt = p000 + (c & 4 ? gyz : 0) + (c & 2 ? gz : 0) + (c & 1);
        const unsigned char* src = base + pt * 64;
        asm("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
            : "=r"(tap[c].v[0]), "=r"(tap[c].v[1]), "=r"(tap[c].v[2]), "=r"(tap[c].v[3]), "=r"(tap[c].v[4]), "=r"(tap[c].v[5]),
              "=r"(tap[c].v[6]), "=r"(tap[c].v[7])
            : "l"(src));
      }
      float acc[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) acc[e] = 0.0f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float w = wx[(c >> 2) & 1] * wy[(c >> 1) & 1] * wz[c & 1];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float2 f = __half22float2(as_h2(tap[c].v[e]));
          acc[2 * e] = fmaf(w, f.x, acc[2 * e]);
          acc[2 * e + 1] = fmaf(w, f.y, acc[2 * e + 1]);
        }
      }
      if (half == 0) {  // (compile-time indices on either side of a warp-uniform branch: v stays in registers)
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = __float_as_uint(acc[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) v[14 + e] = __float_as_uint(acc[e]);
      }
      PROF_MARK(0);
    } else {
    // ---- gather: this half's rounds of products -> tensor memory ------------------------------------------
      // (Gathering a group's NEXT tile into registers in the shadows of the current tile's GEMMs instead was
      // measured slower, 19.6 against 17.6 ms per frame: the GEMMs fetch their weights through the same
      // L1 / shared-memory port the gather saturates, so the two do not overlap.)
      {
        // the sampler's own arithmetic for the position (gnr_sample_t, gnr_point), then normalize_coord
        const float t = POINTS ? 0.0f : gnr_sample_t(p, cur.t_min, cur.k);
        float x = POINTS ? cur.o[0] : gnr_normalize(gnr_point(cur.o[0], cur.d[0], t), p.lo[0], p.inv[0]);
        float y = POINTS ? cur.o[1] : gnr_normalize(gnr_point(cur.o[1], cur.d[1], t), p.lo[1], p.inv[1]);
        const float z = POINTS ? cur.o[2] : gnr_normalize(gnr_point(cur.o[2], cur.d[2], t), p.lo[2], p.inv[2]);
        if (!POINTS && a.blk_px > 0) block_local((float)a.blk_bx, (float)a.blk_by, a.blk_pw, a.blk_ph, x, y, x, y);
        auto taps_of = [&](int pi) -> PairTapsH2 {
          const GnrPlane& pl = planes.p[pi];
          if (NP == 3) {
            const Tap tx = make_tap(x, planes.p[0].fw, planes.p[0].W);
            const Tap ty = make_tap(y, planes.p[0].fh, planes.p[0].H);
            const Tap tz = make_tap(z, planes.p[0].fl, planes.p[0].L);
            return pi == 0 ? make_pair_taps_h2(pl, tx, ty, tz) : (pi == 1 ? make_pair_taps_h2(pl, tx, tz, ty) : make_pair_taps_h2(pl, ty, tz, tx));
          }
          const float u = pick(x, y, z, pl.mat0), v = pick(x, y, z, pl.mat1), l = pick(x, y, z, pl.vec);
          return make_pair_taps_h2(pl, make_tap(u, pl.fw, pl.W), make_tap(v, pl.fh, pl.H), make_tap(l, pl.fl, pl.L));
        };
        auto do_round = [&](int r, const PairTapsH2& t_pair) {  // r is a compile-time constant after inlining
          const int pi = r / 3, g = r - 3 * pi;
          uint32_t q[8];
          if (pi < planes.n) {
            pair_round_h2(planes.p[pi], t_pair, g, q);
          } else {  // fewer than three pairs: these columns are zero
  #pragma unroll
            for (int e = 0; e < 8; ++e) q[e] = 0u;
          }
          tmem_st8(a_tmem + lane_off + r * 8, q);
        };
        // round r = 3 pair + g fills columns 8 r .. 8 r + 7; half 0 takes rounds 0..4, half 1 rounds 5..8
        if (half == 0) {  // (warp-uniform)
          const PairTapsH2 t0 = taps_of(0);
          do_round(0, t0);
          do_round(1, t0);
          do_round(2, t0);
          const PairTapsH2 t1 = taps_of(planes.n > 1 ? 1 : 0);
          do_round(3, t1);
          do_round(4, t1);
        } else {
          const PairTapsH2 t1 = taps_of(planes.n > 1 ? 1 : 0);
          do_round(5, t1);
          const PairTapsH2 t2 = taps_of(planes.n > 2 ? 2 : 0);
          do_round(6, t2);
          do_round(7, t2);
          do_round(8, t2);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      GROUP_SYNC();
      PROF_MARK(0);
  
      // ---- F = A0 * Wb^T (issued by warp 0 of the group) -----------------------------------------------------
      if (wg == 0) {
        tc_fence_after();
        // (no accumulator within the wait limit: nothing is issued or committed, and the group's own wait expires)
        const uint32_t leader = acquire_d() ? elect_one() : 0u;
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
      WAIT_OR_STOP();
      PROF_MARK(2);
      tmem_ld32(f_tmem + lane_off, v);
      tmem_ld_wait();
    }

    // ---- A1: this half's 40 columns of the layer-1 input (K order of the permuted W1 image) -----------------
    {
      uint32_t h[40];
      if (half == 0) {
        // columns 0..6: f0..f13; 7: the constant 1 that multiplies b1; 8..21: (sin f, sin 2f); 22..35: (cos f, cos 2f); 36..39: 0
#pragma unroll
        for (int c = 0; c < 7; ++c) h[c] = pack_h2(__uint_as_float(v[2 * c]), __uint_as_float(v[2 * c + 1]));
        h[7] = pack_h2(1.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < 14; ++i) {  // sin/cos of f and 2 f: one sincos, then the double-angle identities
          float s, c;
          sincos_reduced(__uint_as_float(v[i]), s, c);
          h[8 + i] = pack_h2(s, 2.0f * s * c);
          h[22 + i] = pack_h2(c, 1.0f - 2.0f * s * s);
        }
#pragma unroll
        for (int c = 36; c < 40; ++c) h[c] = 0u;
      } else {
        // columns 40..47: f14..f26, view; 48..60: sin pairs of f14..f26; 61..73: cos pairs; 74..76 / 77..79: view sin / cos pairs
        float val[16];
#pragma unroll
        for (int i = 0; i < 13; ++i) val[i] = __uint_as_float(v[14 + i]);
        val[13] = cur.d[0];
        val[14] = cur.d[1];
        val[15] = cur.d[2];
#pragma unroll
        for (int c = 0; c < 8; ++c) h[c] = pack_h2(val[2 * c], val[2 * c + 1]);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float s, c;
          sincos_reduced(val[i], s, c);
          const uint32_t sp = pack_h2(s, 2.0f * s * c), cp = pack_h2(c, 1.0f - 2.0f * s * s);
          if (i < 13) {
            h[8 + i] = sp;
            h[21 + i] = cp;
          } else {
            h[34 + (i - 13)] = sp;
            h[37 + (i - 13)] = cp;
          }
        }
      }
      const uint32_t at = a_tmem + lane_off + (half ? 40u : 0u);
      tmem_st32(at, *reinterpret_cast<uint32_t(*)[32]>(&h[0]));
      tmem_st8(at + 32, *reinterpret_cast<uint32_t(*)[8]>(&h[32]));
    }
    tmem_st_wait();
    tc_fence_before();
    GROUP_SYNC();
    PROF_MARK(3);

    // ---- D = A1 * W1^T (warp 1) ------------------------------------------------------------------------------
    if (wg == 1) {
      tc_fence_after();
      const uint32_t leader = (SRC == 0 || acquire_d()) ? elect_one() : 0u;  // SRC != 0: no projection came before  // (without a projection this is the tile's first MMA)
#pragma unroll
      for (int ks = 0; ks < K1 / 16; ++ks)
        mma_f16_ts(d_tmem, a_tmem + ks * 8, make_desc(w1_addr + ks * 2 * KG_BYTES, KG_BYTES), kIdescHid, ks > 0 ? 1u : 0u, leader);
      // (test hook of the lattice form, which has no projection GEMM to leave uncommitted)
      const bool skip1 = SRC != 0 && a.debug_skip_commit != 0 && blockIdx.x == 0 && slot == 0 && tile == t_beg;
      mma_commit(mbar, skip1 ? 0u : leader);
      __syncwarp();
    }
    PROF_MARK(4);
    WAIT_OR_STOP();
    PROF_MARK(5);

    // ---- A2 = relu(D) (D already holds b1): half h converts columns 64 h .. 64 h + 63 --------------------------
#pragma unroll
    for (int cb = 0; cb < 2; ++cb) {
      uint32_t v[32];
      tmem_ld32(d_tmem + lane_off + half * 64 + cb * 32, v);
      tmem_ld_wait();
      uint32_t h[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) h[e] = pack_h2_relu(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
      tmem_st16(a_tmem + lane_off + half * 32 + cb * 16, h);
    }
    if (half == 1) {
      const uint32_t tail[8] = {pack_h2(1.0f, 0.0f), 0u, 0u, 0u, 0u, 0u, 0u, 0u};  // k = 128 is the bias input, 129..143 padding
      tmem_st8(a_tmem + lane_off + HID / 2, tail);
    }
    tmem_st_wait();
    tc_fence_before();
    GROUP_SYNC();
    PROF_MARK(6);

    // ---- D = A2 * W2^T (warp 2) ------------------------------------------------------------------------------
    if (wg == 2) {
      tc_fence_after();
      const uint32_t leader = elect_one();
#pragma unroll
      for (int ks = 0; ks < K2 / 16; ++ks)
        mma_f16_ts(d_tmem, a_tmem + ks * 8, make_desc(w2_addr + ks * 2 * KG_BYTES, KG_BYTES), kIdescHid, ks > 0 ? 1u : 0u, leader);
      mma_commit(mbar, leader);
      __syncwarp();
    }
    PROF_MARK(7);
    WAIT_OR_STOP();
    PROF_MARK(8);

    // ---- A3 = relu(D), rgb = sigmoid(A3 * W3^T + b3) (warp 3) ---------------------------------------------------
#pragma unroll
    for (int cb = 0; cb < 2; ++cb) {
      uint32_t v[32];
      tmem_ld32(d_tmem + lane_off + half * 64 + cb * 32, v);
      tmem_ld_wait();
      uint32_t h[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) h[e] = pack_h2_relu(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
      tmem_st16(a_tmem + lane_off + half * 32 + cb * 16, h);
    }
    tmem_st_wait();
    tc_fence_before();
    GROUP_SYNC();
    PROF_MARK(9);
    if (wg == 3) {
      tc_fence_after();
      const uint32_t leader = elect_one();
#pragma unroll
      for (int ks = 0; ks < HID / 16; ++ks)
        mma_f16_ts(f_tmem, a_tmem + ks * 8, make_desc(w3_addr + ks * 2 * KG3_BYTES, KG3_BYTES), kIdescOut, ks > 0 ? 1u : 0u, leader);
      mma_commit(mbar, leader);
      __syncwarp();
    }
    PROF_MARK(10);
    WAIT_OR_STOP();
    PROF_MARK(11);
    if (half == 0) {
      uint32_t r[4];
      tmem_ld4(f_tmem + lane_off, r);
      tmem_ld_wait();
      // the accumulator goes to the tile after the next as soon as its last result is in registers
      tc_fence_before();
      if (FG > 2 && (tid & 31) == 0) asm volatile("red.release.cta.shared::cta.add.u32 [%0], 1;" ::"r"(rel) : "memory");
      if (live) {
        float* out = a.rgb_out + (size_t)j * 3;
        out[0] = 1.0f / (1.0f + __expf(-(s_b3[0] + __uint_as_float(r[0]))));
        out[1] = 1.0f / (1.0f + __expf(-(s_b3[1] + __uint_as_float(r[1]))));
        out[2] = 1.0f / (1.0f + __expf(-(s_b3[2] + __uint_as_float(r[2]))));
      }
    }
    tc_fence_before();  // this tile's tensor-memory reads come before the next tile's writes
    PROF_MARK(12);
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
    if (wg == 0) {
      const uint32_t leader = elect_one();
      mma_commit(mbar, leader);
      __syncwarp();
    }
    group_wait(mbar, parity, bar_id, tg, s_flag, a.wait_limit, GT);
  }
#undef GROUP_SYNC
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS));
  }
}

constexpr size_t kFusedSmem = (size_t)WB_BYTES + W1_BYTES + W2_BYTES + W3_BYTES + 4 * sizeof(float) + MAX_FG * sizeof(uint64_t) + 64;

}  // namespace

// Input column of MLP layer 1 that sits at position k of the fused kernel's A1 operand
// (0..149 = an input of the layer, -2 = the constant 1 that multiplies b1, -1 = zero padding).
void gnr_fused_k1_order(int* map) {
  for (int k = 0; k < K1; ++k) map[k] = -1;
  const int sin0 = APP + 3, cos0 = sin0 + 2 * APP, vsin0 = cos0 + 2 * APP, vcos0 = vsin0 + 6;
  // half 0: columns 0..39
  for (int i = 0; i < 14; ++i) map[i] = i;                       // f0..f13
  map[14] = -2;                                                  // bias input
  for (int i = 0; i < 14; ++i)
    for (int o = 0; o < 2; ++o) {
      map[16 + 2 * i + o] = sin0 + 2 * i + o;
      map[44 + 2 * i + o] = cos0 + 2 * i + o;
    }
  // half 1: columns 40..79
  for (int m = 0; m < 16; ++m) map[80 + m] = m < 13 ? 14 + m : APP + (m - 13);  // f14..f26, view
  for (int i = 14; i < APP; ++i)
    for (int o = 0; o < 2; ++o) {
      map[96 + 2 * (i - 14) + o] = sin0 + 2 * i + o;
      map[122 + 2 * (i - 14) + o] = cos0 + 2 * i + o;
    }
  for (int i = 0; i < 3; ++i)
    for (int o = 0; o < 2; ++o) {
      map[148 + 2 * i + o] = vsin0 + 2 * i + o;
      map[154 + 2 * i + o] = vcos0 + 2 * i + o;
    }
}

int gnr_app_fusable(const GnrModel* m) {
  // with the appearance lattice the planes' storage type does not matter: they are not read
  if (m->app_lattice && m->cfg.mlp_mode == 2 && m->cfg.unfused_appearance == 0) return 1;
  // fp16 appearance planes of 48 (padded) channels, the single-fp16 tensor-core mode, and a product count
  // that fits the 80 operand columns
  return m->cfg.mlp_mode == 2 && m->cfg.app_storage == 1 && m->cfg.unfused_appearance != 1 && gnr_tc_basis_fused(m) &&
         m->app[0].C == 48 && m->mlp.n_prod == m->cfg.n_pairs * 48 && m->mlp.n_prod <= MAX_K0;
}

int launch_app_mlp_fused(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, float* rgb, int32_t* status,
                         cudaStream_t st, const float* features, int feat_stride, const void* parts_h, int n_parts,
                         int64_t part_stride_rows) {
  if (parts_h) features = reinterpret_cast<const float*>(parts_h);  // (marks the features-given family below)
  if (!m->mlp.tc_image) {
    gnr_set_error("tensor-core MLP weights were not prepared");
    return -1;
  }
  const bool points = c.xyz_direct != nullptr || features != nullptr;
  if (features ? (!c.view_direct) : (c.xyz_direct ? (!c.view_direct) : (!c.ids || c.index || (!c.total_ptr && c.total_direct <= 0)))) {
    gnr_set_error("the fused appearance kernel walks an appearance list (ids + device count), explicit points with view "
                  "directions, or explicit features with view directions");
    return -1;
  }
  PlaneSet set = make_set(m->app, m->cfg.n_pairs);
  FusedArgs a;
  a.rays = c.rays;
  a.t_min = c.t_min;
  a.ids = c.ids;
  a.total_ptr = c.total_ptr;
  a.total_direct = c.total_direct;
  a.capacity = c.capacity;
  a.xyz_direct = c.xyz_direct ? c.xyz_direct : c.view_direct;  // (with given features the position is never read)
  a.view_direct = c.view_direct;
  a.point_stride = c.point_stride;
  a.w_image = (const unsigned char*)m->mlp.tc_image;
  a.b3 = m->mlp.b3;
  a.rgb_out = rgb;
  a.status = status;
  a.k0 = m->mlp.n_prod;
  a.wait_limit = m->debug_wait_limit > 0 ? (uint32_t)m->debug_wait_limit : kWaitLimit;
  a.debug_skip_commit = m->debug_expire_wait;
  a.prof = m->debug_prof;
  a.lat = (const unsigned char*)m->app_lattice;
  for (int i = 0; i < 3; ++i) a.lat_g[i] = m->app_lat_dims[i];
  a.feat = features;
  a.feat_stride = feat_stride;
  a.parts = (const unsigned char*)parts_h;
  a.n_parts = n_parts;
  a.part_stride = part_stride_rows;
  a.blk_px = points ? 0 : c.blk_px;
  a.blk_bx = c.blk_bx;
  a.blk_by = c.blk_by;
  a.blk_pw = c.blk_pw;
  a.blk_ph = c.blk_ph;
  auto launch = [&](auto kernel, int groups) -> int {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFusedSmem);
    if (e != cudaSuccess) return (int)e;
    kernel<<<m->sm_count, groups * GT, kFusedSmem, st>>>(p, set, a);
    return 0;
  };
  auto pick_variant = [&](auto groups_tag) -> int {
    constexpr int G = decltype(groups_tag)::value;
    if (parts_h) return launch(app_mlp_fused_kernel<3, false, true, 3, G>, G);
    if (features) return launch(app_mlp_fused_kernel<3, false, true, 2, G>, G);
    if (m->app_lattice)  // features from the projected-feature lattice: no gather of planes, no projection GEMM
      return points ? launch(app_mlp_fused_kernel<3, false, true, 1, G>, G) : launch(app_mlp_fused_kernel<3, false, false, 1, G>, G);
    if (points)
      return standard_vm3(set) ? launch(app_mlp_fused_kernel<3, false, true, 0, G>, G)
                               : launch(app_mlp_fused_kernel<0, false, true, 0, G>, G);
    if (a.prof)
      return standard_vm3(set) ? launch(app_mlp_fused_kernel<3, true, false, 0, G>, G)
                               : launch(app_mlp_fused_kernel<0, true, false, 0, G>, G);
    return standard_vm3(set) ? launch(app_mlp_fused_kernel<3, false, false, 0, G>, G)
                             : launch(app_mlp_fused_kernel<0, false, false, 0, G>, G);
  };
  const int rc = m->cfg.unfused_appearance == 3 ? pick_variant(std::integral_constant<int, 2>{})
                                                : pick_variant(std::integral_constant<int, 3>{});
  if (rc) return rc;
  return (int)cudaGetLastError();
}
