// Partial basis projection of a CHANNEL SLICE of the appearance field at explicit points, fp16 out.
//
// Tensor (channel) parallel rendering (app/models/gridnerf_tensor_parallel.py:198-217,284-330): every rank
// holds a slice of the appearance channels of every plane and line and the matching columns of basis_mat,
// and contributes, for every appearance sample of the group, the partial sum
//   F_r = basis[:, slice_r] * (plane x line products of slice_r)            (27 values per sample)
// which are then summed over the ranks.  This kernel computes F_r for points that any rank sampled.
//
// Same construction as the first two steps of the one-kernel appearance path (gnr_app_fused.cu): the
// products of a 128-point tile go from registers straight into tensor memory (tcgen05.st) and are the A
// operand of one small GEMM (M 128, N 32, K = 3 pairs x padded channels) against the basis image in shared
// memory; the 32 fp32 result columns are read back, rounded to fp16 and stored as one 64-byte row per point
// (the transport format of the exchange that follows: half the bytes of fp32, and the sum over the ranks is
// taken in fp32 by the receiver).  A slice has 16, 32 or 48 padded channels per pair (RP = 1, 2, 3 rounds of
// 16), stored as fp16 texels of 32 RP bytes.
//
// One persistent CTA per SM; a group of 128 threads (thread = row = lane of tensor memory) owns 24 RP + 32
// columns of tensor memory and works on its own tiles: nothing is shared between groups, so six groups
// (four for RP = 3) keep six tiles in flight.  Every wait on an mbarrier is bounded (status word
// GNR_ST_WAIT_EXPIRED, then the group stops, commits once more and waits before the CTA frees tensor memory).
#include "gnr_gather.cuh"
#include "gnr_tc.cuh"

namespace {

constexpr int ST = 128;  // threads per group

struct SliceArgs {
  const float* xyz;             // [n][stride] normalised positions
  int stride;
  long long n;
  const unsigned char* basis;   // fp16 operand image of the basis: [k group][32 rows][8] (gnr_mlp_tc_prepare)
  unsigned char* out;           // [n][32] fp16
  int32_t* status;
  uint32_t wait_limit;
  int debug_skip_commit;        // test hook: group 0 of CTA 0 leaves out the commit of its first GEMM
};

template <int RP>
__device__ __forceinline__ H16 ldg_h16_slice(const void* base, uint32_t texel, int g) {
  const unsigned char* ptr = reinterpret_cast<const unsigned char*>(base) + (size_t)texel * (uint32_t)(RP * 32) + g * 32;
  H16 r;
  asm("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7])
      : "l"(ptr));
  return r;
}

// pair_round_h2 (gnr_gather.cuh) for texels of RP * 16 channels
template <int RP>
__device__ __forceinline__ void slice_round_h2(const GnrPlane& pl, const PairTapsH2& t, int g, uint32_t (&q)[8]) {
  const H16 a = ldg_h16_slice<RP>(pl.plane, t.nw, g), b = ldg_h16_slice<RP>(pl.plane, t.nw + 1u, g);
  const H16 c = ldg_h16_slice<RP>(pl.plane, t.sw, g), d = ldg_h16_slice<RP>(pl.plane, t.sw + 1u, g);
  const H16 l0 = ldg_h16_slice<RP>(pl.line, t.seg, g), l1 = ldg_h16_slice<RP>(pl.line, t.seg + 1u, g);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    __half2 pv = __hmul2(as_h2(a.v[e]), t.w_nw);
    pv = __hfma2(as_h2(b.v[e]), t.w_ne, pv);
    pv = __hfma2(as_h2(c.v[e]), t.w_sw, pv);
    pv = __hfma2(as_h2(d.v[e]), t.w_se, pv);
    const __half2 lv = __hfma2(as_h2(l1.v[e]), t.h_l1, __hmul2(as_h2(l0.v[e]), t.h_l0));
    q[e] = as_u32(__hmul2(pv, lv));
  }
}

template <int RP>
struct SliceGeom {
  static constexpr int kGroups = RP == 3 ? 4 : 6;
  static constexpr int kACols = 3 * RP * 8;      // products of a row: 3 pairs x RP rounds x 8 columns (16 fp16)
  static constexpr int kCols = kACols + NB;      // + the fp32 result
  static constexpr int kSteps = 3 * RP;          // MMAs (K = 16 each) per tile
};

template <int RP>
__global__ void __launch_bounds__(SliceGeom<RP>::kGroups * ST, 1) app_slice_project_kernel(PlaneSet planes, SliceArgs a) {
  using G = SliceGeom<RP>;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* s_wb = smem;                                                       // kSteps * 2 k groups of 512 bytes
  uint64_t* s_mbar = reinterpret_cast<uint64_t*>(s_wb + G::kSteps * 2 * KGB_BYTES);  // [groups] MMA completion
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_mbar + G::kGroups);
  volatile uint32_t* s_flag = s_tmem + 1;                                           // [groups] outcome of a group's last wait

  const int tid = threadIdx.x, warp = tid >> 5;
  const int warp_u = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int slot = warp_u >> 2, row = tid & (ST - 1);
  const bool lead_warp = (warp_u & 3) == 0;
  {
    const uint4* src = reinterpret_cast<const uint4*>(a.basis);
    uint4* dst = reinterpret_cast<uint4*>(s_wb);
    for (int i = tid; i < G::kSteps * 2 * KGB_BYTES / 16; i += G::kGroups * ST) dst[i] = src[i];
    if (tid == 0) {
      for (int s = 0; s < G::kGroups; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_mbar[s])));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
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
  const uint32_t a_tmem = tmem_base + (uint32_t)(slot * G::kCols);
  const uint32_t f_tmem = a_tmem + (uint32_t)G::kACols;
  const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
  const uint32_t wb_addr = smem_u32(s_wb);
  const uint32_t mbar = smem_u32(&s_mbar[slot]);
  const int bar_id = 1 + slot;
  s_flag += slot;
  uint32_t parity = 0;
  bool expired = false;

  const long long n_tiles = (a.n + ROWS - 1) / ROWS;
  const long long per = (n_tiles + gridDim.x - 1) / gridDim.x;
  const long long t_beg = min(n_tiles, (long long)blockIdx.x * per), t_end = min(n_tiles, t_beg + per);

  for (long long tile = t_beg + slot; tile < t_end; tile += G::kGroups) {
    const long long j_raw = tile * ROWS + row;
    const bool live = j_raw < a.n;
    const long long j = live ? j_raw : a.n - 1;  // rows past the end repeat the last point and write nothing
    {
      const float* src = a.xyz + (size_t)j * a.stride;
      const float x = __ldg(src + 0), y = __ldg(src + 1), z = __ldg(src + 2);
#pragma unroll
      for (int pi = 0; pi < 3; ++pi) {
        if (pi < planes.n) {
          const GnrPlane& pl = planes.p[pi];
          const float u = pick(x, y, z, pl.mat0), v = pick(x, y, z, pl.mat1), l = pick(x, y, z, pl.vec);
          const PairTapsH2 t = make_pair_taps_h2(pl, make_tap(u, pl.fw, pl.W), make_tap(v, pl.fh, pl.H), make_tap(l, pl.fl, pl.L));
#pragma unroll
          for (int g = 0; g < RP; ++g) {
            uint32_t q[8];
            slice_round_h2<RP>(pl, t, g, q);
            tmem_st8(a_tmem + lane_off + (pi * RP + g) * 8, q);
          }
        } else {  // fewer than three pairs: these columns are zero
          const uint32_t zero[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
          for (int g = 0; g < RP; ++g) tmem_st8(a_tmem + lane_off + (pi * RP + g) * 8, zero);
        }
      }
    }
    tmem_st_wait();
    tc_fence_before();
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
    if (lead_warp) {
      tc_fence_after();
      const uint32_t leader = elect_one();
#pragma unroll
      for (int ks = 0; ks < G::kSteps; ++ks)
        mma_f16_ts(f_tmem, a_tmem + ks * 8, make_desc(wb_addr + ks * 2 * KGB_BYTES, KGB_BYTES), kIdescBasis, ks > 0 ? 1u : 0u, leader);
      const bool skip = a.debug_skip_commit != 0 && blockIdx.x == 0 && slot == 0 && tile == t_beg;
      mma_commit(mbar, skip ? 0u : leader);
      __syncwarp();
    }
    if (!group_wait(mbar, parity, bar_id, row, s_flag, a.wait_limit)) {
      if (row == 0) atomicExch(a.status + GNR_ST_WAIT_EXPIRED, 1);
      expired = true;
      break;
    }
    parity ^= 1;
    uint32_t v[32];
    tmem_ld32(f_tmem + lane_off, v);
    tmem_ld_wait();
    if (live) {
      uint4* dst = reinterpret_cast<uint4*>(a.out + (size_t)j * 64);
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        uint4 o;
        o.x = pack_h2(__uint_as_float(v[8 * q4 + 0]), __uint_as_float(v[8 * q4 + 1]));
        o.y = pack_h2(__uint_as_float(v[8 * q4 + 2]), __uint_as_float(v[8 * q4 + 3]));
        o.z = pack_h2(__uint_as_float(v[8 * q4 + 4]), __uint_as_float(v[8 * q4 + 5]));
        o.w = pack_h2(__uint_as_float(v[8 * q4 + 6]), __uint_as_float(v[8 * q4 + 7]));
        dst[q4] = o;
      }
    }
    tc_fence_before();  // this tile's tensor-memory reads come before the next tile's writes
  }
  if (expired) {
    if (lead_warp) {
      const uint32_t leader = elect_one();
      mma_commit(mbar, leader);
      __syncwarp();
    }
    group_wait(mbar, parity, bar_id, row, s_flag, a.wait_limit);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u));
  }
}

// out[i][c] = sum over the W parts of part[w][i][c] (fp16 rows of 32), c < n_out, accumulated in fp32
__global__ void __launch_bounds__(256) sum_partials_kernel(const unsigned char* __restrict__ parts, int n_parts, long long rows,
                                                           long long part_stride_rows, int n_out, int out_stride,
                                                           float* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (row, group of 8 columns)
  if (i >= rows * 4) return;
  const long long r = i >> 2;
  const int cg = (int)(i & 3);
  float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
  for (int w = 0; w < n_parts; ++w) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(parts + ((size_t)w * part_stride_rows + r) * 64) + cg);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __half22float2(as_h2(u[e]));
      acc[2 * e] += f.x;
      acc[2 * e + 1] += f.y;
    }
  }
  float* dst = out + (size_t)r * out_stride;
#pragma unroll
  for (int e = 0; e < 8; ++e)
    if (cg * 8 + e < n_out) dst[cg * 8 + e] = acc[e];
}

template <int RP>
int launch_slice(const GnrModel* m, const PlaneSet& set, const SliceArgs& a, cudaStream_t st) {
  using G = SliceGeom<RP>;
  const size_t smem = (size_t)G::kSteps * 2 * KGB_BYTES + G::kGroups * sizeof(uint64_t) + 64;
  cudaError_t e = cudaFuncSetAttribute(app_slice_project_kernel<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  app_slice_project_kernel<RP><<<m->sm_count, G::kGroups * ST, smem, st>>>(set, a);
  return (int)cudaGetLastError();
}

}  // namespace

int launch_app_slice_project(const GnrModel* m, const float* xyz, int stride, int64_t n, void* features_h, int32_t* status,
                             cudaStream_t st) {
  const int cp = m->app[0].C;  // padded channels per pair
  if (m->cfg.mlp_mode != 2 || m->cfg.app_storage != 1 || !m->mlp.tc_image || m->cfg.n_pairs > 3 || m->cfg.app_dim > APP ||
      (cp != 16 && cp != 32 && cp != 48)) {
    gnr_set_error("slice projection needs mlp_mode 2, fp16 appearance planes (app_storage 1) of at most 48 channels, at most "
                  "three pairs and app_dim <= 27 (got mode %d, storage %d, %d padded channels, %d pairs, app_dim %d)",
                  m->cfg.mlp_mode, m->cfg.app_storage, cp, m->cfg.n_pairs, m->cfg.app_dim);
    return -1;
  }
  PlaneSet set = make_set(m->app, m->cfg.n_pairs);
  SliceArgs a;
  a.xyz = xyz;
  a.stride = stride;
  a.n = n;
  a.basis = (const unsigned char*)m->mlp.tc_image;
  a.out = (unsigned char*)features_h;
  a.status = status;
  a.wait_limit = m->debug_wait_limit > 0 ? (uint32_t)m->debug_wait_limit : kWaitLimit;
  a.debug_skip_commit = m->debug_expire_wait;
  return cp == 16 ? launch_slice<1>(m, set, a, st) : (cp == 32 ? launch_slice<2>(m, set, a, st) : launch_slice<3>(m, set, a, st));
}

int launch_sum_partials(const void* parts_h, int n_parts, int64_t rows, int64_t part_stride_rows, int n_out, int out_stride,
                        float* out, cudaStream_t st) {
  if (rows <= 0) return 0;
  const long long threads = rows * 4;
  sum_partials_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>((const unsigned char*)parts_h, n_parts, rows,
                                                                        part_stride_rows, n_out, out_stride, out);
  return (int)cudaGetLastError();
}
