// Ray generation, sampling + occupancy test, exclusive scan, compaction.
//
// Bit-exactness contract of the sampler: the set of valid (ray, sample) pairs equals what
// the torch renderer selects (sample_ray, app/models/gridnerf_sequential.py:260-281, then the
// alphaMask filter :460-465 with AlphaGridMask.sample_alpha, app/models/alpha_mask.py:35-59).
// Every floating-point operation below is therefore a single correctly rounded IEEE
// operation (__fadd_rn/__fmul_rn/__fdiv_rn are never contracted into FMAs), in the order
// in which torch's separate elementwise kernels apply them.
#include "gnr_internal.cuh"

namespace {

constexpr int kWarpsPerBlock = 8;

// ---------------------------------------------------------------------------------------------
// ray generation: d = (dir_x[i], dir_y[j], -1) @ R^T, o = c2w[:, 3]
// (dist_render/dataset/utils.py:57-89)
// ---------------------------------------------------------------------------------------------
struct Pose {
  float m[12];
};

__global__ void raygen_kernel(Pose pose, const float* __restrict__ dir_x, const float* __restrict__ dir_y,
                              int W, const int32_t* __restrict__ pixel_ids, int64_t first_pixel, int64_t n,
                              float* __restrict__ rays) {
  int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  int64_t pix = pixel_ids ? (int64_t)pixel_ids[r] : first_pixel + r;
  int j = (int)(pix / W), i = (int)(pix - (int64_t)j * W);
  float dx = dir_x[i], dy = dir_y[j], dz = -1.0f;
  float* out = rays + r * 6;
  out[0] = pose.m[3];
  out[1] = pose.m[7];
  out[2] = pose.m[11];
#pragma unroll
  for (int a = 0; a < 3; ++a)
    out[3 + a] = fmaf(dz, pose.m[a * 4 + 2], fmaf(dy, pose.m[a * 4 + 1], dx * pose.m[a * 4 + 0]));
}

// Same, with the pose read from device memory: a captured CUDA graph replays this launch for a new
// pose by rewriting those 12 floats.
__global__ void raygen_dev_kernel(const float* __restrict__ pose_dev, const float* __restrict__ dir_x,
                                  const float* __restrict__ dir_y, int W, const int32_t* __restrict__ pixel_ids,
                                  int64_t first_pixel, int64_t n, float* __restrict__ rays) {
  int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  float m[12];
#pragma unroll
  for (int i = 0; i < 12; ++i) m[i] = __ldg(pose_dev + i);
  int64_t pix = pixel_ids ? (int64_t)pixel_ids[r] : first_pixel + r;
  int j = (int)(pix / W), i = (int)(pix - (int64_t)j * W);
  float dx = dir_x[i], dy = dir_y[j], dz = -1.0f;
  float* out = rays + r * 6;
  out[0] = m[3];
  out[1] = m[7];
  out[2] = m[11];
#pragma unroll
  for (int a = 0; a < 3; ++a) out[3 + a] = fmaf(dz, m[a * 4 + 2], fmaf(dy, m[a * 4 + 1], dx * m[a * 4 + 0]));
}

// ---------------------------------------------------------------------------------------------
// sampling: one thread per ray, samples in order, 32 validity bits per register word
// ---------------------------------------------------------------------------------------------
// AlphaGridMask.sample_alpha (app/models/alpha_mask.py:35-59): trilinear interpolation of the 0/1
// volume with zero padding, then `> threshold`.  The sum runs over the corners in grid_sample's
// order with individually rounded operations.  Two exact shortcuts come first: a clear bit of the
// coarse grid proves that all eight corners are empty (threshold >= 0 then fails), and with a
// threshold of exactly zero the sum of non-negative weights is positive as soon as one occupied
// corner has a positive weight, so the loop can stop there.
// `skip` (optional): when the coarse grids decide the sample (empty block: invalid; full block and
// threshold 0: valid), the number of FOLLOWING samples that provably lie in the same block and so
// get the same answer, given the index-space step `di` per sample
// (dense sampler: positions advance by d * stepSize).  The bound keeps 1/100 of a mask cell away
// from the block's faces, far more than the rounding of the index arithmetic (a few 1e-4).
__device__ __forceinline__ bool occupancy_test(const GnrSampleParams& p, float px, float py, float pz,
                                               const float* di = nullptr, int* skip = nullptr) {
  // q = (p - aabb0) * invgridSize - 1 ; index = ((q + 1) / 2) * (size - 1)
  const float ix = __fmul_rn(__fmul_rn(__fadd_rn(gnr_normalize(px, p.a_lo[0], p.a_inv[0]), 1.0f), 0.5f), (float)(p.aW - 1));
  const float iy = __fmul_rn(__fmul_rn(__fadd_rn(gnr_normalize(py, p.a_lo[1], p.a_inv[1]), 1.0f), 0.5f), (float)(p.aH - 1));
  const float iz = __fmul_rn(__fmul_rn(__fadd_rn(gnr_normalize(pz, p.a_lo[2], p.a_inv[2]), 1.0f), 0.5f), (float)(p.aD - 1));
  // corners outside the volume contribute zero (padding_mode="zeros"); indices that do not
  // fit an int (only possible for samples far outside the mask box) are outside too.
  const bool okx = (ix >= -1.0f) && (ix < (float)p.aW), oky = (iy >= -1.0f) && (iy < (float)p.aH),
             okz = (iz >= -1.0f) && (iz < (float)p.aD);
  if (!(okx && oky && okz)) return 0.0f > p.a_thres;
  const float fx0 = floorf(ix), fy0 = floorf(iy), fz0 = floorf(iz);
  const int x0 = (int)fx0, y0 = (int)fy0, z0 = (int)fz0;
  if (p.a_coarse != nullptr && p.a_thres >= 0.0f && x0 >= 0 && y0 >= 0 && z0 >= 0) {
    const uint32_t cb = (uint32_t)(((z0 >> 2) * p.cH + (y0 >> 2)) * p.cW + (x0 >> 2));
    const uint32_t cw = cb >> 5, cs = cb & 31;
    const bool empty = !((__ldg(p.a_coarse + cw) >> cs) & 1u);
    // a full block decides the test when the threshold is exactly zero: the lower corner is occupied
    // and its weight (x0 + 1 - ix)(y0 + 1 - iy)(z0 + 1 - iz) is a product of three positive floats
    const bool full = !empty && p.a_thres == 0.0f && ((__ldg(p.a_full + cw) >> cs) & 1u);
    if (empty || full) {
      if (skip) {
        const float idx[3] = {ix, iy, iz};
        const int lo[3] = {x0 & ~3, y0 & ~3, z0 & ~3};
        float n = 64.0f;
#pragma unroll
        for (int a = 0; a < 3; ++a) {
          const float room = di[a] > 0.0f ? ((float)(lo[a] + 4) - idx[a] - 0.01f) : (idx[a] - (float)lo[a] - 0.01f);
          const float speed = fabsf(di[a]);
          if (speed > 0.0f) n = fminf(n, room / speed);
        }
        *skip = n > 0.0f ? (int)n : 0;
      }
      return full;
    }
  }
  const float fx1 = __fadd_rn(fx0, 1.0f), fy1 = __fadd_rn(fy0, 1.0f), fz1 = __fadd_rn(fz0, 1.0f);
  const float wx[2] = {__fsub_rn(fx1, ix), __fsub_rn(ix, fx0)};
  const float wy[2] = {__fsub_rn(fy1, iy), __fsub_rn(iy, fy0)};
  const float wz[2] = {__fsub_rn(fz1, iz), __fsub_rn(iz, fz0)};
  const bool stop_at_first = p.a_thres == 0.0f;
  float out = 0.0f;
#pragma unroll
  for (int cz = 0; cz < 2; ++cz) {
#pragma unroll
    for (int cy = 0; cy < 2; ++cy) {
      const int y = y0 + cy, z = z0 + cz;
      if ((unsigned)y >= (unsigned)p.aH || (unsigned)z >= (unsigned)p.aD) continue;
      const uint32_t row = (uint32_t)((z * p.aH + y) * p.aW);
#pragma unroll
      for (int cx = 0; cx < 2; ++cx) {
        const int x = x0 + cx;
        if ((unsigned)x < (unsigned)p.aW) {
          const uint32_t bit = row + (uint32_t)x;
          if ((__ldg(p.a_bits + (bit >> 5)) >> (bit & 31)) & 1u) {
            const float w = __fmul_rn(__fmul_rn(wx[cx], wy[cy]), wz[cz]);
            out = __fadd_rn(out, w);  // tap is exactly 1, so tap * w == w
            if (stop_at_first && w > 0.0f) return true;
          }
        }
      }
    }
  }
  return out > p.a_thres;
}

constexpr int kSampleBlock = 128;

__global__ void __launch_bounds__(kSampleBlock)
sample_mask_kernel(GnrSampleParams p, const float* __restrict__ rays, int64_t n_rays, float* __restrict__ t_min_out,
                   uint32_t* __restrict__ words_out, int32_t* __restrict__ counts_out) {
  const int64_t ray_raw = (int64_t)blockIdx.x * kSampleBlock + threadIdx.x;
  const bool live = ray_raw < n_rays;  // lanes past the end keep their warp company (warp votes below) and write nothing
  const int64_t ray = live ? ray_raw : n_rays - 1;
  const float* r = rays + ray * 6;
  const float o[3] = {__ldg(r), __ldg(r + 1), __ldg(r + 2)};
  const float d[3] = {__ldg(r + 3), __ldg(r + 4), __ldg(r + 5)};
  // slab entry: max over axes of min(rate_a, rate_b), clamped to [near, far]
  float t_min = -INFINITY;
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    const float vec = (d[a] == 0.0f) ? 1e-6f : d[a];
    const float ra = __fdiv_rn(__fsub_rn(p.hi[a], o[a]), vec);
    const float rb = __fdiv_rn(__fsub_rn(p.lo[a], o[a]), vec);
    t_min = fmaxf(t_min, fminf(ra, rb));
  }
  t_min = fminf(fmaxf(t_min, p.near_t), p.far_t);
  if (p.mode == 1) {
    // hull sampler: the per-ray parameter is `far`, the hit with the ground plane z = aabb_min_z
    // (far = -(o_z - z0) / d_z, replaced by near_far[1] for rays that do not point down)
    const float far = -__fdiv_rn(__fsub_rn(o[2], p.lo[2]), d[2]);
    t_min = (d[2] >= 0.0f) ? p.far_t : far;
  }
  if (live) t_min_out[ray] = t_min;

  int count = 0;
  uint32_t* wrow = words_out + ray * p.words;
  // fl(o + fl(d * fl(t_min + fl(step * k)))) is monotone in k, so once a sample has left the
  // box through the far side of an axis every later sample is outside as well.
  // (The hull sampler's distances are a sum of a falling and a rising term and need not be
  // monotone to the last bit, so only the dense sampler stops at the first exit and skips.)
  // The 32 rays of a warp walk the sample index k together.  When every ray of the warp stands in
  // an empty coarse block (or has left the box) the warp jumps over the samples that all of them
  // can rule out; jumping together keeps neighbouring rays, which see the same occupancy, in step.
  const float di[3] = {d[0] * p.step * p.a_inv[0] * 0.5f * (float)(p.aW - 1), d[1] * p.step * p.a_inv[1] * 0.5f * (float)(p.aH - 1),
                       d[2] * p.step * p.a_inv[2] * 0.5f * (float)(p.aD - 1)};
  const bool can_skip = p.mode == 0 && p.has_mask;
  constexpr int kMaxSkip = 64;
  // Samples that are skipped as VALID (full blocks) must also lie inside the box: they do while their
  // index stays two samples short of the slab exit (the positions are monotone along the ray and the
  // sample that started the run was tested inside).
  int k_inside = -1;
  if (can_skip) {
    float t_far = INFINITY;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
      if (d[a] != 0.0f) t_far = fminf(t_far, fmaxf((p.hi[a] - o[a]) / d[a], (p.lo[a] - o[a]) / d[a]));
    }
    const float ksafe = floorf((t_far - t_min) / p.step) - 2.0f;
    k_inside = ksafe > 0.0f ? (int)fminf(ksafe, (float)p.S) : -1;
  }
  bool done = !live;
  uint32_t bits = 0;
  int word = 0, k = 0;
  int ones_beg = 0, ones_end = 0;  // samples [ones_beg, ones_end) of this ray are valid without a test
  auto with_ones = [&](uint32_t b, int wd) {
    const int lo = max(ones_beg, wd * 32), hi = min(ones_end, wd * 32 + 32);
    if (lo < hi) b |= (hi - lo == 32 ? 0xffffffffu : ((1u << (hi - lo)) - 1u)) << (lo - wd * 32);
    return b;
  };
  while (k < p.S) {
    const int w = k >> 5;
    while (word < w) {  // words completed since the last sample (all of them when samples were skipped)
      bits = with_ones(bits, word);
      if (live) wrow[word] = bits;
      ++word;
      count += __popc(bits);
      bits = 0;
    }
    int skip = kMaxSkip;  // a finished ray never holds the warp back
    bool run_valid = false;
    if (!done) {
      skip = 0;
      const float t = gnr_sample_t(p, t_min, k);
      const float px = gnr_point(o[0], d[0], t), py = gnr_point(o[1], d[1], t), pz = gnr_point(o[2], d[2], t);
      const bool lo_out = (p.lo[0] > px) | (p.lo[1] > py) | (p.lo[2] > pz);
      const bool hi_out = (px > p.hi[0]) | (py > p.hi[1]) | (pz > p.hi[2]);
      if (!(lo_out | hi_out)) {
        if (!p.has_mask || occupancy_test(p, px, py, pz, di, can_skip ? &skip : nullptr)) {
          bits |= 1u << (k & 31);
          run_valid = true;
          skip = max(0, min(skip, k_inside - k));  // a run of valid samples ends before the box does
        }
      } else if (p.mode == 0) {
        const bool exited = ((d[0] > 0.0f) & (px > p.hi[0])) | ((d[0] < 0.0f) & (p.lo[0] > px)) |
                            ((d[1] > 0.0f) & (py > p.hi[1])) | ((d[1] < 0.0f) & (p.lo[1] > py)) |
                            ((d[2] > 0.0f) & (pz > p.hi[2])) | ((d[2] < 0.0f) & (p.lo[2] > pz)) |
                            ((d[0] == 0.0f) & ((p.lo[0] > px) | (px > p.hi[0]))) |
                            ((d[1] == 0.0f) & ((p.lo[1] > py) | (py > p.hi[1]))) |
                            ((d[2] == 0.0f) & ((p.lo[2] > pz) | (pz > p.hi[2])));
        if (exited) {
          done = true;
          skip = kMaxSkip;
        }
      }
    }
    if (__all_sync(0xffffffffu, done)) break;
    const int jump = __reduce_min_sync(0xffffffffu, min(skip, kMaxSkip));
    if (run_valid && jump > 0) {  // (jump > 0 implies this lane's own run is at least that long)
      bits = with_ones(bits, w);  // what an earlier run left in the current word, before the range moves on
      ones_beg = k + 1;
      ones_end = min(k + 1 + jump, p.S);
    }
    k += 1 + jump;
  }
  while (word < p.words) {
    bits = with_ones(bits, word);
    if (live) wrow[word] = bits;
    ++word;
    count += __popc(bits);
    bits = 0;
  }
  if (live) counts_out[ray] = count;
}

// ---------------------------------------------------------------------------------------------
// exclusive scan of int32 (three small kernels, no inter-block waits)
// ---------------------------------------------------------------------------------------------
constexpr int kScanBlock = 1024;

__device__ __forceinline__ int block_exclusive_scan(int v, int* total) {
  __shared__ int warp_sums[32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sums[wid] = incl;
  __syncthreads();
  if (wid == 0) {
    int s = warp_sums[lane];
    int si = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, si, o);
      if (lane >= o) si += t;
    }
    warp_sums[lane] = si - s;  // exclusive warp base
    if (lane == 31) *total = si;
  }
  __syncthreads();
  int res = warp_sums[wid] + incl - v;
  __syncthreads();
  return res;
}

__global__ void __launch_bounds__(kScanBlock)
scan_local_kernel(const int32_t* __restrict__ in, int32_t* __restrict__ out, int32_t* __restrict__ block_sums, int64_t n) {
  __shared__ int total;
  int64_t i = (int64_t)blockIdx.x * kScanBlock + threadIdx.x;
  int v = (i < n) ? in[i] : 0;
  int ex = block_exclusive_scan(v, &total);
  if (i < n) out[i] = ex;
  if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kScanBlock)
scan_sums_kernel(int32_t* __restrict__ block_sums, int n_blocks, int32_t* __restrict__ out_total,
                 int32_t* __restrict__ status, int total_slot, int overflow_slot, long long capacity) {
  __shared__ int total;
  long long carry = 0;
  for (int base = 0; base < n_blocks; base += kScanBlock) {
    int i = base + threadIdx.x;
    int v = (i < n_blocks) ? block_sums[i] : 0;
    int ex = block_exclusive_scan(v, &total);
    if (i < n_blocks) block_sums[i] = (int)(carry + ex);
    carry += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    *out_total = (int)carry;
    status[total_slot] = (int)carry;
    status[overflow_slot] = (carry > capacity) ? 1 : 0;
  }
}

__global__ void __launch_bounds__(kScanBlock)
scan_add_kernel(int32_t* __restrict__ out, const int32_t* __restrict__ block_sums, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * kScanBlock + threadIdx.x;
  if (i < n) out[i] += block_sums[blockIdx.x];
}

// ---------------------------------------------------------------------------------------------
// compaction: ids[offsets[ray] + rank of sample among the ray's valid ones] = ray << kbits | k
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
expand_ids_kernel(const uint32_t* __restrict__ words, const int32_t* __restrict__ offsets, int64_t n_rays, int n_words,
                  int kbits, long long capacity, uint32_t* __restrict__ ids) {
  const int lane = threadIdx.x & 31;
  int64_t ray = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (ray >= n_rays) return;
  long long pos = offsets[ray];
  long long end = offsets[ray + 1];
  if (pos == end) return;
  const uint32_t* wrow = words + ray * n_words;
  for (int w = 0; w < n_words && pos < end; ++w) {
    uint32_t bits = __ldg(wrow + w);
    if ((bits >> lane) & 1u) {
      long long at = pos + __popc(bits & ((1u << lane) - 1u));
      if (at < capacity) ids[at] = ((uint32_t)ray << kbits) | (uint32_t)(w * 32 + lane);
    }
    pos += __popc(bits);
  }
}

}  // namespace

int launch_exclusive_scan(const int32_t* counts, int32_t* offsets, int32_t* block_sums, int64_t n,
                          int32_t* status, int total_slot, int overflow_slot, int64_t capacity,
                          cudaStream_t st) {
  int n_blocks = (int)((n + kScanBlock - 1) / kScanBlock);
  if (n_blocks < 1) n_blocks = 1;
  scan_local_kernel<<<n_blocks, kScanBlock, 0, st>>>(counts, offsets, block_sums, n);
  scan_sums_kernel<<<1, kScanBlock, 0, st>>>(block_sums, n_blocks, offsets + n, status, total_slot, overflow_slot,
                                             (long long)capacity);
  scan_add_kernel<<<n_blocks, kScanBlock, 0, st>>>(offsets, block_sums, n);
  return (int)cudaGetLastError();
}

int launch_sample_mask(const GnrModel* m, const GnrSampleParams& p, const float* rays, int64_t n, char* ws,
                       const GnrWs& L, cudaStream_t st) {
  (void)m;
  unsigned blocks = (unsigned)((n + kSampleBlock - 1) / kSampleBlock);
  sample_mask_kernel<<<blocks, kSampleBlock, 0, st>>>(p, rays, n, (float*)(ws + L.t_min), (uint32_t*)(ws + L.words),
                                                            (int32_t*)(ws + L.counts));
  return (int)cudaGetLastError();
}

int launch_sample_compact(const GnrModel* m, const GnrSampleParams& p, int64_t n, char* ws, const GnrWs& L,
                          int64_t max_valid, int with_ids, cudaStream_t st) {
  (void)m;
  int32_t* offsets = (int32_t*)(ws + L.offsets);
  int e = launch_exclusive_scan((const int32_t*)(ws + L.counts), offsets, (int32_t*)(ws + L.block_sums), n,
                                (int32_t*)(ws + L.status), GNR_ST_NUM_VALID, GNR_ST_OVERFLOW_VALID, max_valid, st);
  if (e || !with_ids) return e;  // the fused march pass and the appearance compaction read the words themselves
  unsigned blocks = (unsigned)((n + kWarpsPerBlock - 1) / kWarpsPerBlock);
  expand_ids_kernel<<<blocks, kWarpsPerBlock * 32, 0, st>>>((const uint32_t*)(ws + L.words), offsets, n, p.words, p.kbits,
                                                           (long long)max_valid, (uint32_t*)(ws + L.ids));
  return (int)cudaGetLastError();
}

extern "C" int gnr_generate_rays(const float* pose_h, const float* dir_x, const float* dir_y, int H, int W,
                                 const int32_t* pixel_ids, int64_t first_pixel, int64_t n, float* rays,
                                 void* stream) {
  if (!pose_h || !dir_x || !dir_y || !rays || H <= 0 || W <= 0 || n < 0) {
    gnr_set_error("gnr_generate_rays: bad argument");
    return -1;
  }
  if (!pixel_ids && (first_pixel < 0 || first_pixel + n > (int64_t)H * W)) {
    gnr_set_error("gnr_generate_rays: pixel range [%lld, %lld) outside the %dx%d image", (long long)first_pixel,
                  (long long)(first_pixel + n), W, H);
    return -1;
  }
  if (n == 0) return 0;
  Pose p;
  for (int i = 0; i < 12; ++i) p.m[i] = pose_h[i];
  raygen_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(p, dir_x, dir_y, W, pixel_ids,
                                                                              first_pixel, n, rays);
  GNR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int gnr_generate_rays_dev(const float* pose_dev, const float* dir_x, const float* dir_y, int H, int W,
                                     const int32_t* pixel_ids, int64_t first_pixel, int64_t n, float* rays,
                                     void* stream) {
  if (!pose_dev || !dir_x || !dir_y || !rays || H <= 0 || W <= 0 || n < 0) {
    gnr_set_error("gnr_generate_rays_dev: bad argument");
    return -1;
  }
  if (!pixel_ids && (first_pixel < 0 || first_pixel + n > (int64_t)H * W)) {
    gnr_set_error("gnr_generate_rays_dev: pixel range [%lld, %lld) outside the %dx%d image", (long long)first_pixel,
                  (long long)(first_pixel + n), W, H);
    return -1;
  }
  if (n == 0) return 0;
  raygen_dev_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(pose_dev, dir_x, dir_y, W, pixel_ids,
                                                                                  first_pixel, n, rays);
  GNR_CUDA_OK(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free sampling: same kernels, scratch in a fixed device array of this library.
// ---------------------------------------------------------------------------------------------
// Scratch of gnr_sample_static: [validity bit words][scan block sums].  One copy per GPU that
// loads the library, shared by every call on that GPU.
static __device__ __align__(256) unsigned char g_sample_static_scratch[GNR_SAMPLE_STATIC_SCRATCH_BYTES];

#include <mutex>

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
unsigned char* g_static_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on `device`.  The array's name is only a host-side
// handle; the address a kernel can use comes from cudaGetSymbolAddress, asked once per
// device with that device current.
int static_scratch_for(int device, unsigned char** out) {
  if (device < 0 || device >= kMaxDevices) {
    gnr_set_error("gnr_sample_static: device ordinal %d outside [0, %d)", device, kMaxDevices);
    return -1;
  }
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_ptr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_sample_static_scratch);
    if (e != cudaSuccess || !p) {
      gnr_set_error("gnr_sample_static: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
      return -2;
    }
    g_static_ptr[device] = (unsigned char*)p;
  }
  *out = g_static_ptr[device];
  return 0;
}

inline size_t round256(size_t v) { return (v + 255) / 256 * 256; }
}  // namespace

extern "C" int gnr_sample_static(GnrModel* m, const float* rays, int64_t n_rays, int n_samples, int64_t max_valid,
                                 float* t_min, int32_t* counts, int32_t* offsets, uint32_t* ids, int32_t* status,
                                 void* stream) {
  if (!m) {
    gnr_set_error("gnr_sample_static: null model");
    return -1;
  }
  if (!rays || !t_min || !counts || !offsets || !ids || !status) {
    gnr_set_error("gnr_sample_static: rays and all five output buffers are required");
    return -1;
  }
  if (n_rays < 1 || n_samples < 1 || max_valid < 1) {
    gnr_set_error("gnr_sample_static: bad sizes (n_rays %lld, n_samples %d, max_valid %lld)", (long long)n_rays, n_samples,
                  (long long)max_valid);
    return -1;
  }
  // the same sampler preconditions gnr_sample checks (hull tables present and of this length)
  if (gnr_check_sampler(m, n_samples)) return -1;
  const int kbits = gnr_sample_bits(n_samples);
  if (kbits > 20 || n_rays > ((int64_t)1 << (32 - kbits)) || n_rays * (int64_t)n_samples > 0x7fffffffLL ||
      max_valid > 0x7fffffffLL) {
    gnr_set_error("gnr_sample_static: %lld rays x %d samples does not fit the 32-bit sample ids", (long long)n_rays, n_samples);
    return -1;
  }
  const size_t words = (size_t)(n_samples + 31) / 32;
  const size_t words_bytes = round256((size_t)n_rays * words * 4);
  const size_t sums_bytes = round256(((size_t)n_rays / 1024 + 2) * 4);
  if (words_bytes + sums_bytes > (size_t)GNR_SAMPLE_STATIC_SCRATCH_BYTES) {
    gnr_set_error("gnr_sample_static: %lld rays x %d samples need %zu bytes of scratch, the built-in array holds %u; "
                  "split the chunk or use gnr_sample with a workspace",
                  (long long)n_rays, n_samples, words_bytes + sums_bytes, (unsigned)GNR_SAMPLE_STATIC_SCRATCH_BYTES);
    return -1;
  }
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != m->device) cudaSetDevice(m->device);
  unsigned char* scratch = nullptr;
  int rc = static_scratch_for(m->device, &scratch);
  if (rc == 0) {
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t* mask_words = (uint32_t*)scratch;
    int32_t* block_sums = (int32_t*)(scratch + words_bytes);
    GnrSampleParams p = gnr_sample_params(m, n_samples);
    const unsigned blocks = (unsigned)((n_rays + kWarpsPerBlock - 1) / kWarpsPerBlock);
    cudaError_t e = cudaMemsetAsync(status, 0, GNR_ST_WORDS * sizeof(int32_t), st);  // the overflow flag starts at zero
    if (e == cudaSuccess) {
      // every word of mask_words and block_sums that is read below is written first by these
      // launches, so what an earlier call left in the array is never seen
      sample_mask_kernel<<<(unsigned)((n_rays + kSampleBlock - 1) / kSampleBlock), kSampleBlock, 0, st>>>(p, rays, n_rays, t_min,
                                                                                                  mask_words, counts);
      e = (cudaError_t)launch_exclusive_scan(counts, offsets, block_sums, n_rays, status, GNR_ST_NUM_VALID,
                                             GNR_ST_OVERFLOW_VALID, max_valid, st);
    }
    if (e == cudaSuccess) {
      expand_ids_kernel<<<blocks, kWarpsPerBlock * 32, 0, st>>>(mask_words, offsets, n_rays, p.words, p.kbits,
                                                               (long long)max_valid, ids);
      e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
      gnr_set_error("gnr_sample_static: launch failed: %s", cudaGetErrorString(e));
      rc = -2;
    }
  }
  if (prev != m->device) cudaSetDevice(prev);
  return rc;
}
