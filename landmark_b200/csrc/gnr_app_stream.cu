// Appearance gather + basis projection + MLP in one kernel, producer / consumer form.
//
// Same arithmetic, operand layouts and weight images as app_mlp_fused_kernel (gnr_app_fused.cu; the
// reference code it stands for is named there).  What differs is who does what:
//
//   warps 8..15  PRODUCER: gather only.  For tile after tile they interpolate the plane x line
//                products (two threads per row, nine rounds of 16 channels split 5 / 4) and write
//                them with tcgen05.st into one of three operand buffers in tensor memory.  The L1
//                port therefore works all the time, not only in a group's gather phase.
//   warps 0..7   CONSUMER: everything after the gather, for TWO tiles at a time.  A tile goes through
//                five phases, each starting with a wait for the tile's previous GEMM:
//                  0  products ready (producer) -> issue F = A0 * Wb^T
//                  1  F -> positional encoding -> A1 -> issue D = A1 * W1^T
//                  2  relu(D) -> A2 -> issue D = A2 * W2^T
//                  3  relu(D) -> A3 -> issue out = A3 * W3^T
//                  4  out -> sigmoid -> rgb; the operand buffer goes back to the producer
//                and the consumer alternates between its two tiles phase by phase, so the CUDA-core
//                work of one tile runs while the GEMM of the other is in the tensor pipe.
//
// Tensor memory (512 columns): accumulators D0, D1 (128 each) of the two tile slots; operand buffers
// A0, A1, A2 (80 each): tile i uses slot i % 2 and buffer i % 3 (products, then A1, A2, A3 of the same
// tile in place).  The projection's 32 result columns and layer 3's 16 are the first columns of the
// slot's accumulator, which is idle at those times.
//
// Synchronisation: full[b] (8 producer warps arrive, consumer waits), empty[b] (consumer arrives after
// the tile's last GEMM, producer waits), mma[s] (tcgen05.commit of slot s).  Every wait is bounded; a
// wait that runs out raises status[GNR_ST_WAIT_EXPIRED] and a shared abort flag that both roles check
// at every tile, and before the tensor memory is freed one thread commits once more and waits
// (bounded) so that no GEMM of the CTA is still running.
#include "gnr_gather.cuh"
#include "gnr_tc.cuh"

namespace {

constexpr int CT = 256;                 // consumer threads (warps 0..7), two per row
constexpr int PT = 256;                 // producer threads (warps 8..15), two per row
constexpr int D_COLS = HID;             // per tile slot
constexpr int A_COLS = 80;              // per operand buffer
constexpr int A_BASE = 2 * D_COLS;      // first operand buffer
constexpr int N_ABUF = 3;

struct StreamArgs {
  const float* rays;             // [n][6]
  const float* t_min;            // [n]
  const uint32_t* ids;           // appearance list: ray << kbits | sample
  const int32_t* total_ptr;      // length of the list (device)
  long long capacity;
  const unsigned char* w_image;  // [basis][W1][W2][W3][W1 with permuted K] fp16 operand images
  const float* b3;
  float* rgb_out;
  int32_t* status;
  int k0;                        // products per sample (n_pairs * 48)
  uint32_t wait_limit;           // polls a bounded wait may take
  int debug_skip_commit;         // test hook: the first projection of CTA 0 is never committed
};

struct RowRay {  // what a row needs of its list entry
  float o[3], d[3], t_min;
  int k;
};

__device__ __forceinline__ void mbar_arrive(uint32_t mbar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar) : "memory");
}

template <int NP>
__global__ void __launch_bounds__(CT + PT, 1) app_mlp_stream_kernel(GnrSampleParams p, PlaneSet planes, StreamArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* s_wb = smem;
  unsigned char* s_w1 = s_wb + WB_BYTES;  // layer 1 with the permuted K order (gnr_fused_k1_order)
  unsigned char* s_w2 = s_w1 + W1_BYTES;
  unsigned char* s_w3h = s_w2 + W2_BYTES;
  float* s_b3 = reinterpret_cast<float*>(s_w3h + W3_BYTES);
  uint64_t* s_full = reinterpret_cast<uint64_t*>(s_b3 + 4);  // [3]
  uint64_t* s_empty = s_full + N_ABUF;                       // [3]
  uint64_t* s_mma = s_empty + N_ABUF;                        // [2]
  uint64_t* s_drain = s_mma + 2;                             // [1]
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_drain + 1);
  volatile uint32_t* s_flag = s_tmem + 1;   // outcome of the consumer's last wait
  volatile uint32_t* s_abort = s_tmem + 2;  // set by whichever role gave up

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int warp_u = __shfl_sync(0xffffffffu, tid >> 5, 0);  // the same number, known to be warp-uniform
  const bool producer = warp_u >= CT / 32;
  const int wr = warp_u & 7;       // warp within its role
  const int half = wr >> 2;        // which half of every row's columns this thread takes
  const int row = tid & 127;

  {
    const uint4* src = reinterpret_cast<const uint4*>(a.w_image);
    const uint4* src_w1p = reinterpret_cast<const uint4*>(a.w_image + WB_BYTES + W1_BYTES + W2_BYTES + W3_BYTES);
    uint4* dst = reinterpret_cast<uint4*>(s_wb);
    constexpr int kAll = (WB_BYTES + W1_BYTES + W2_BYTES + W3_BYTES) / 16, kW1Beg = WB_BYTES / 16, kW1End = (WB_BYTES + W1_BYTES) / 16;
    for (int i = tid; i < kAll; i += CT + PT) dst[i] = (i >= kW1Beg && i < kW1End) ? src_w1p[i - kW1Beg] : src[i];
    if (tid < 4) s_b3[tid] = a.b3[tid];
    if (tid == 0) {
      for (int b = 0; b < N_ABUF; ++b) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&s_full[b])), "r"(PT / 32));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_empty[b])));
      }
      for (int s = 0; s < 2; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_mma[s])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(s_drain)), "r"(CT / 32));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      *s_abort = 0u;
    }
    if (warp == 0) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(512u));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *s_tmem, 0);
  const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;  // the lane quarter this warp may touch
  const uint32_t wb_addr = smem_u32(s_wb), w1_addr = smem_u32(s_w1), w2_addr = smem_u32(s_w2), w3_addr = smem_u32(s_w3h);

  const long long total = min((long long)*a.total_ptr, a.capacity);
  const long long n_tiles_all = (total + ROWS - 1) / ROWS;
  // a contiguous share of the list per CTA: neighbouring tiles are neighbouring rays, whose texels are
  // still in this SM's L1
  const long long per = (n_tiles_all + gridDim.x - 1) / gridDim.x;
  const long long t_beg = min(n_tiles_all, (long long)blockIdx.x * per), t_end = min(n_tiles_all, t_beg + per);
  const int n_tiles = (int)(t_end - t_beg);

  if (producer) {
    // =========================================== PRODUCER ===========================================
    const uint32_t kmask = (1u << p.kbits) - 1u;
    auto entry_of = [&](int i) -> uint32_t {  // list entry of this thread's row in tile i of the CTA
      const long long jr = (t_beg + i) * ROWS + row;
      return __ldg(a.ids + (jr < total ? jr : total - 1));  // rows past the end repeat the last entry
    };
    auto load_ray = [&](uint32_t id) -> RowRay {
      RowRay r;
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
    // the entry of a row is fetched two tiles ahead and its ray one tile ahead
    uint32_t id_ahead = 0;
    RowRay next_ray = {};
    if (n_tiles > 0) next_ray = load_ray(entry_of(0));
    if (n_tiles > 1) id_ahead = entry_of(1);
    for (int i = 0; i < n_tiles; ++i) {
      if (*s_abort) break;
      const int b = i % N_ABUF;
      const RowRay cur = next_ray;
      if (i + 1 < n_tiles) next_ray = load_ray(id_ahead);
      if (i + 2 < n_tiles) id_ahead = entry_of(i + 2);
      // wait until the tile that used this buffer three tiles ago is finished (the first use of a
      // buffer finds the barrier in its initial phase and passes)
      if (i >= N_ABUF) {
        uint32_t ok = 1u;
        if (lane == 0) ok = mbar_wait_bounded(smem_u32(&s_empty[b]), (uint32_t)((i / N_ABUF - 1) & 1), a.wait_limit) ? 1u : 0u;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          if (lane == 0) {
            atomicExch(a.status + GNR_ST_WAIT_EXPIRED, 1);
            *s_abort = 1u;
          }
          break;
        }
        tc_fence_after();
      }
      // the sampler's own arithmetic for the position (gnr_sample_t, gnr_point), then normalize_coord
      const float t = gnr_sample_t(p, cur.t_min, cur.k);
      const float x = gnr_normalize(gnr_point(cur.o[0], cur.d[0], t), p.lo[0], p.inv[0]);
      const float y = gnr_normalize(gnr_point(cur.o[1], cur.d[1], t), p.lo[1], p.inv[1]);
      const float z = gnr_normalize(gnr_point(cur.o[2], cur.d[2], t), p.lo[2], p.inv[2]);
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
      const uint32_t a_buf = tmem_base + A_BASE + b * A_COLS + lane_off;
      auto do_round = [&](int r, const PairTapsH2& t_pair) {  // round r = 3 pair + g fills columns 8 r .. 8 r + 7
        const int pi = r / 3, g = r - 3 * pi;
        uint32_t q[8];
        if (pi < planes.n) {
          pair_round_h2(planes.p[pi], t_pair, g, q);
        } else {  // fewer than three pairs: these columns are zero
#pragma unroll
          for (int e = 0; e < 8; ++e) q[e] = 0u;
        }
        tmem_st8(a_buf + r * 8, q);
      };
      if (half == 0) {  // (warp-uniform) rounds 0..4
        const PairTapsH2 t0 = taps_of(0);
        do_round(0, t0);
        do_round(1, t0);
        do_round(2, t0);
        const PairTapsH2 t1 = taps_of(planes.n > 1 ? 1 : 0);
        do_round(3, t1);
        do_round(4, t1);
      } else {  // rounds 5..8, and the view direction for the consumer: fp32 bits in columns 76..78
        const PairTapsH2 t1 = taps_of(planes.n > 1 ? 1 : 0);
        do_round(5, t1);
        const PairTapsH2 t2 = taps_of(planes.n > 2 ? 2 : 0);
        do_round(6, t2);
        do_round(7, t2);
        do_round(8, t2);
        const uint32_t vw[4] = {__float_as_uint(cur.d[0]), __float_as_uint(cur.d[1]), __float_as_uint(cur.d[2]), 0u};
        asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(a_buf + 76), "r"(vw[0]), "r"(vw[1]),
                     "r"(vw[2]), "r"(vw[3])
                     : "memory");
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_full[b]));
    }
  } else {
    // =========================================== CONSUMER ===========================================
    const int ct = tid;  // thread within the consumer (0..255)
    int tile_of[2] = {-1, -1}, phase_of[2] = {0, 0};
    uint32_t mma_par[2] = {0u, 0u};
    int next_tile = 0;
    bool stop = false;
    const int ksteps0 = a.k0 >> 4;
#define CONSUMER_SYNC() asm volatile("bar.sync 1, 256;" ::: "memory")
    while (!stop) {
      bool any = false;
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        if (stop) break;
        if (tile_of[s] < 0 && next_tile < n_tiles) {
          tile_of[s] = next_tile++;
          phase_of[s] = 0;
        }
        if (tile_of[s] < 0) continue;
        any = true;
        const int i = tile_of[s], b = i % N_ABUF, ph = phase_of[s];
        const uint32_t d_tmem = tmem_base + s * D_COLS;              // accumulator of this slot
        const uint32_t a_tmem = tmem_base + A_BASE + b * A_COLS;     // operand buffer of this tile
        const uint32_t mbar = smem_u32(&s_mma[s]);
        // ---- every phase starts with a bounded wait: products (phase 0) or the previous GEMM of the tile
        {
          const uint32_t wbar = ph == 0 ? smem_u32(&s_full[b]) : mbar;
          const uint32_t wpar = ph == 0 ? (uint32_t)((i / N_ABUF) & 1) : mma_par[s];
          if (!group_wait(wbar, wpar, 1, ct, s_flag, a.wait_limit, CT) || *s_abort) {
            if (ct == 0) {
              atomicExch(a.status + GNR_ST_WAIT_EXPIRED, 1);
              *s_abort = 1u;
            }
            stop = true;
            break;
          }
          if (ph != 0) mma_par[s] ^= 1u;
        }
        const int issuer = (ph + 4 * s) & 7;  // the warp that issues this phase's GEMM: spread over the consumer's warps
        if (ph == 0) {
          // ---- F = A0 * Wb^T into the first 32 columns of the slot's accumulator --------------------------
          if (wr == issuer) {
            tc_fence_after();
            const uint32_t leader = elect_one();
#pragma unroll
            for (int ks = 0; ks < MAX_K0 / 16; ++ks) {
              if (ks < ksteps0)
                mma_f16_ts(d_tmem, a_tmem + ks * 8, make_desc(wb_addr + ks * 2 * KGB_BYTES, KGB_BYTES), kIdescBasis, ks > 0 ? 1u : 0u, leader);
            }
            const bool skip = a.debug_skip_commit != 0 && blockIdx.x == 0 && i == 0;
            mma_commit(mbar, skip ? 0u : leader);
            __syncwarp();
          }
        } else if (ph == 1) {
          // ---- A1: this half's 40 columns of the layer-1 input (K order of the permuted W1 image) ---------
          uint32_t v[32];  // the 27 projected features of this row (columns 27..31 are zero padding)
          tmem_ld32(d_tmem + lane_off, v);
          uint32_t vw[4] = {0u, 0u, 0u, 0u};
          if (half == 1)
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];\n"
                         : "=r"(vw[0]), "=r"(vw[1]), "=r"(vw[2]), "=r"(vw[3])
                         : "r"(a_tmem + lane_off + 76));
          tmem_ld_wait();
          tc_fence_before();
          CONSUMER_SYNC();  // every thread has read the view columns before half 1 overwrites them with A1
          uint32_t h[40];
          if (half == 0) {
            // columns 0..6: f0..f13; 7: the constant 1 that multiplies b1; 8..21: (sin f, sin 2f); 22..35: (cos f, cos 2f); 36..39: 0
#pragma unroll
            for (int c = 0; c < 7; ++c) h[c] = pack_h2(__uint_as_float(v[2 * c]), __uint_as_float(v[2 * c + 1]));
            h[7] = pack_h2(1.0f, 0.0f);
#pragma unroll
            for (int k = 0; k < 14; ++k) {  // sin/cos of f and 2 f: one sincos, then the double-angle identities
              float sn, cs;
              sincos_reduced(__uint_as_float(v[k]), sn, cs);
              h[8 + k] = pack_h2(sn, 2.0f * sn * cs);
              h[22 + k] = pack_h2(cs, 1.0f - 2.0f * sn * sn);
            }
#pragma unroll
            for (int c = 36; c < 40; ++c) h[c] = 0u;
          } else {
            // columns 40..47: f14..f26, view; 48..60: sin pairs of f14..f26; 61..73: cos pairs; 74..76 / 77..79: view sin / cos pairs
            float val[16];
#pragma unroll
            for (int k = 0; k < 13; ++k) val[k] = __uint_as_float(v[14 + k]);
            val[13] = __uint_as_float(vw[0]);
            val[14] = __uint_as_float(vw[1]);
            val[15] = __uint_as_float(vw[2]);
#pragma unroll
            for (int c = 0; c < 8; ++c) h[c] = pack_h2(val[2 * c], val[2 * c + 1]);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              float sn, cs;
              sincos_reduced(val[k], sn, cs);
              const uint32_t sp = pack_h2(sn, 2.0f * sn * cs), cp = pack_h2(cs, 1.0f - 2.0f * sn * sn);
              if (k < 13) {
                h[8 + k] = sp;
                h[21 + k] = cp;
              } else {
                h[34 + (k - 13)] = sp;
                h[37 + (k - 13)] = cp;
              }
            }
          }
          const uint32_t at = a_tmem + lane_off + (half ? 40u : 0u);
          tmem_st32(at, *reinterpret_cast<uint32_t(*)[32]>(&h[0]));
          tmem_st8(at + 32, *reinterpret_cast<uint32_t(*)[8]>(&h[32]));
          tmem_st_wait();
          tc_fence_before();
          CONSUMER_SYNC();
          if (wr == issuer) {
            tc_fence_after();
            const uint32_t leader = elect_one();
#pragma unroll
            for (int ks = 0; ks < K1 / 16; ++ks)
              mma_f16_ts(d_tmem, a_tmem + ks * 8, make_desc(w1_addr + ks * 2 * KG_BYTES, KG_BYTES), kIdescHid, ks > 0 ? 1u : 0u, leader);
            mma_commit(mbar, leader);
            __syncwarp();
          }
        } else if (ph == 2 || ph == 3) {
          // ---- relu(D) -> A2 resp. A3 (D already holds the bias): half h converts columns 64 h .. 64 h + 63 -----
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
          if (ph == 2 && half == 1) {
            const uint32_t tail[8] = {pack_h2(1.0f, 0.0f), 0u, 0u, 0u, 0u, 0u, 0u, 0u};  // k = 128 is the bias input, 129..143 padding
            tmem_st8(a_tmem + lane_off + HID / 2, tail);
          }
          tmem_st_wait();
          tc_fence_before();
          CONSUMER_SYNC();
          if (wr == issuer) {
            tc_fence_after();
            const uint32_t leader = elect_one();
            if (ph == 2) {
#pragma unroll
              for (int ks = 0; ks < K2 / 16; ++ks)
                mma_f16_ts(d_tmem, a_tmem + ks * 8, make_desc(w2_addr + ks * 2 * KG_BYTES, KG_BYTES), kIdescHid, ks > 0 ? 1u : 0u, leader);
            } else {
#pragma unroll
              for (int ks = 0; ks < HID / 16; ++ks)
                mma_f16_ts(d_tmem, a_tmem + ks * 8, make_desc(w3_addr + ks * 2 * KG3_BYTES, KG3_BYTES), kIdescOut, ks > 0 ? 1u : 0u, leader);
            }
            mma_commit(mbar, leader);
            __syncwarp();
          }
        } else {
          // ---- rgb = sigmoid(out + b3); the operand buffer returns to the producer -----------------------------
          if (ct == 0) mbar_arrive(smem_u32(&s_empty[b]));  // the tile's last GEMM has completed: nothing reads the buffer any more
          if (half == 0) {
            uint32_t r[4];
            tmem_ld4(d_tmem + lane_off, r);
            tmem_ld_wait();
            const long long j = (t_beg + i) * ROWS + row;
            if (j < total) {
              float* out = a.rgb_out + (size_t)j * 3;
              out[0] = 1.0f / (1.0f + __expf(-(s_b3[0] + __uint_as_float(r[0]))));
              out[1] = 1.0f / (1.0f + __expf(-(s_b3[1] + __uint_as_float(r[1]))));
              out[2] = 1.0f / (1.0f + __expf(-(s_b3[2] + __uint_as_float(r[2]))));
            }
          }
          tc_fence_before();  // (the next tile of this slot starts with a wait + barrier before anything writes D)
        }
        phase_of[s] = ph + 1;
        if (ph == 4) tile_of[s] = -1;
      }
      if (!any && next_tile >= n_tiles) break;
    }
#undef CONSUMER_SYNC
  }

  // ---- teardown ---------------------------------------------------------------------------------------------
  if (!producer && *s_abort) {
    // GEMMs may still be running: every consumer warp commits once more (a commit covers the GEMMs its own
    // elected lane issued) and warp 0 waits (bounded) for all of them before the tensor memory goes
    const uint32_t leader = elect_one();
    mma_commit(smem_u32(s_drain), leader);
    __syncwarp();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    if (*s_abort) {
      if (lane == 0) mbar_wait_bounded(smem_u32(s_drain), 0u, a.wait_limit);
      __syncwarp();
    }
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u));
  }
}

constexpr size_t kStreamSmem = (size_t)WB_BYTES + W1_BYTES + W2_BYTES + W3_BYTES + 4 * sizeof(float) + 9 * sizeof(uint64_t) + 64;

}  // namespace

int launch_app_mlp_stream(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, float* rgb, int32_t* status,
                          cudaStream_t st) {
  if (!m->mlp.tc_image) {
    gnr_set_error("tensor-core MLP weights were not prepared");
    return -1;
  }
  if (!c.ids || c.index || c.xyz_direct || !c.total_ptr) {
    gnr_set_error("the fused appearance kernel walks an appearance list (ids + device count)");
    return -1;
  }
  PlaneSet set;
  set.n = m->cfg.n_pairs;
  for (int i = 0; i < set.n; ++i) set.p[i] = m->app[i];
  StreamArgs a;
  a.rays = c.rays;
  a.t_min = c.t_min;
  a.ids = c.ids;
  a.total_ptr = c.total_ptr;
  a.capacity = c.capacity;
  a.w_image = (const unsigned char*)m->mlp.tc_image;
  a.b3 = m->mlp.b3;
  a.rgb_out = rgb;
  a.status = status;
  a.k0 = m->mlp.n_prod;
  a.wait_limit = m->debug_wait_limit > 0 ? (uint32_t)m->debug_wait_limit : kWaitLimit;
  a.debug_skip_commit = m->debug_expire_wait;
  cudaError_t e;
  if (standard_vm3(set)) {
    e = cudaFuncSetAttribute(app_mlp_stream_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStreamSmem);
    if (e != cudaSuccess) return (int)e;
    app_mlp_stream_kernel<3><<<m->sm_count, CT + PT, kStreamSmem, st>>>(p, set, a);
  } else {
    e = cudaFuncSetAttribute(app_mlp_stream_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStreamSmem);
    if (e != cudaSuccess) return (int)e;
    app_mlp_stream_kernel<0><<<m->sm_count, CT + PT, kStreamSmem, st>>>(p, set, a);
  }
  return (int)cudaGetLastError();
}
