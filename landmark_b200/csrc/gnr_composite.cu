// Transmittance / weights (raw2alpha), appearance-sample compaction, final compositing.
//
// raw2alpha (app/tools/utils.py:51-64): alpha = 1 - exp(-sigma * dist),
// T = cumprod([1, 1 - alpha + 1e-10]), w = alpha * T[:-1].  Samples that failed the validity
// test have sigma = 0, hence alpha = 0 and a factor of exactly 1.0f, so the product over a
// ray's compacted samples equals the product over all of its samples, taken in sample order as
// torch.cumprod does on the CPU.
#include "gnr_internal.cuh"

namespace {

constexpr int kWarpsPerBlock = 8;

// One thread per ray, samples in order: the same operations in the same order as the fused
// march kernel, so both give the same bits.
__global__ void __launch_bounds__(32)  // one warp per CTA: a finished warp frees its slot at once
weights_kernel(GnrSampleParams p, float distance_scale, float thres, const float* __restrict__ t_min_arr,
               const uint32_t* __restrict__ words, const float* __restrict__ sigma, const int32_t* __restrict__ offsets,
               int64_t n_rays, long long capacity, float* __restrict__ weight, float* __restrict__ acc_out,
               float* __restrict__ depth_out, int32_t* __restrict__ app_counts, const int32_t* __restrict__ rows,
               float2* __restrict__ packed) {
  // `rows`: sigma of list entry i is sigma[rows[i]] (answers of block owners, still in the order they were sent).
  // `packed`: write only the samples above the appearance threshold, as (weight, sample) pairs at the front of the
  // ray's range (the form expand_app_packed_kernel reads); sigma must then not live in the workspace's own arrays.
  const int64_t ray = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (ray >= n_rays) return;
  const long long beg = offsets[ray], end = min((long long)offsets[ray + 1], capacity);
  float acc = 0.0f, dep = 0.0f;
  int n_app = 0;
  if (beg < end) {
    const float t_min = t_min_arr[ray];
    float T = 1.0f;  // transmittance before the current sample
    // entry i of the valid list is the (i - beg)-th set bit of the ray's validity words, in order
    const uint32_t* wrow = words + (size_t)ray * p.words;
    int word = 0;
    uint32_t bits = __ldg(wrow);
    for (long long i = beg; i < end; ++i) {
      while (bits == 0u && word + 1 < p.words) bits = __ldg(wrow + ++word);
      const int k = word * 32 + (__ffs(bits) - 1);
      bits &= bits - 1u;
      const float t = gnr_sample_t(p, t_min, k);
      // dists = z[k+1] - z[k], 0 for the last sample (gridnerf_sequential.py:457)
      const float dist = (k == p.S - 1) ? 0.0f : __fsub_rn(gnr_sample_t(p, t_min, k + 1), t);
      const float sg = __ldg(sigma + (rows ? (long long)__ldg(rows + i) : i));
      const float alpha = __fsub_rn(1.0f, expf(__fmul_rn(-sg, __fmul_rn(dist, distance_scale))));
      const float w = alpha * T;
      if (packed) {
        if (w > thres) packed[beg + n_app] = make_float2(w, __int_as_float(k));
      } else {
        weight[i] = w;
      }
      acc += w;
      dep = fmaf(w, t, dep);
      n_app += (w > thres) ? 1 : 0;
      T *= __fadd_rn(__fsub_rn(1.0f, alpha), 1e-10f);
    }
  }
  acc_out[ray] = acc;
  depth_out[ray] = dep;
  app_counts[ray] = n_app;
}

// Order of the appearance list.  Rays are taken in groups of 32 consecutive rays (one warp, lane =
// ray).  Group g owns positions app_offsets[32 g] .. app_offsets[32 g + 32) of the list (the
// exclusive scan of the per-ray counts); inside the group the samples are ordered by rank first
// and ray second: all first appearance samples of the group's rays, then all second ones, ...
// With rays in tile order the 32 entries a warp of the gather or MLP kernel touches together are
// then samples of neighbouring pixels at about the same depth, which read the same texels, and
// their rows in the product tiles are consecutive.  app_group_walk yields, for rank j, the list
// position of this lane's sample; both kernels below and nothing else define the order.
struct AppGroupWalk {
  long long pos;  // position of rank j of the group's first active ray
  __device__ __forceinline__ bool step(int lane, bool has, long long& at) {
    const uint32_t mask = __ballot_sync(0xffffffffu, has);
    if (mask == 0u) return false;
    at = pos + __popc(mask & ((1u << lane) - 1u));
    pos += __popc(mask);
    return true;
  }
};

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
expand_app_kernel(const float* __restrict__ weight, const uint32_t* __restrict__ words, int n_words, int kbits,
                  float thres, const int32_t* __restrict__ offsets, const int32_t* __restrict__ app_counts,
                  const int32_t* __restrict__ app_offsets, int64_t n_rays, long long capacity, long long app_capacity,
                  int32_t* __restrict__ app_index, uint32_t* __restrict__ app_ids, float* __restrict__ app_weight) {
  const int lane = threadIdx.x & 31;
  const int64_t group = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (group * 32 >= n_rays) return;
  const int64_t ray = group * 32 + lane;
  const bool has_ray = ray < n_rays;
  int left = has_ray ? app_counts[ray] : 0;  // appearance samples this ray still has to place
  long long i = has_ray ? offsets[ray] : 0;
  const long long end = has_ray ? min((long long)offsets[ray + 1], capacity) : 0;
  // entry i of the valid list is the (i - offsets[ray])-th set bit of the ray's validity words
  const uint32_t* wrow = words + (size_t)(has_ray ? ray : 0) * n_words;
  int word = 0;
  uint32_t bits = has_ray ? __ldg(wrow) : 0u;
  AppGroupWalk walk;
  walk.pos = app_offsets[group * 32];
  long long at;
  while (walk.step(lane, left > 0, at)) {
    if (left > 0) {
      float w = 0.0f;
      int k = 0;
      bool found = false;
      while (i < end && !found) {  // the next sample with w > thres
        while (bits == 0u && word + 1 < n_words) bits = __ldg(wrow + ++word);
        k = word * 32 + (__ffs(bits) - 1);
        bits &= bits - 1u;
        w = __ldg(weight + i);
        found = w > thres;
        if (!found) ++i;
      }
      if (found && at < app_capacity) {
        app_index[at] = (int32_t)i;
        app_ids[at] = ((uint32_t)ray << kbits) | (uint32_t)k;  // the gather and MLP kernels find ray and sample here
        app_weight[at] = w;                                     // the compositing reads its weights in list order
      }
      ++i;
      --left;
    }
  }
}

// The same list from the packed output of the march (list_only): ray r's j-th appearance sample is the pair
// (weight, sample number) at packed[offsets[r] + j]; no walk over weights or validity bits.
// (app_index, the valid-list index of an entry, is not produced: nothing in the frame loop reads it.)
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
expand_app_packed_kernel(const float2* __restrict__ packed, int kbits,
                         const int32_t* __restrict__ offsets, const int32_t* __restrict__ app_counts,
                         const int32_t* __restrict__ app_offsets, int64_t n_rays, long long capacity, long long app_capacity,
                         uint32_t* __restrict__ app_ids, float* __restrict__ app_weight) {
  const int lane = threadIdx.x & 31;
  const int64_t group = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (group * 32 >= n_rays) return;
  const int64_t ray = group * 32 + lane;
  const bool has_ray = ray < n_rays;
  int left = has_ray ? app_counts[ray] : 0;
  long long i = has_ray ? offsets[ray] : 0;
  const long long end = has_ray ? min((long long)offsets[ray + 1], capacity) : 0;
  AppGroupWalk walk;
  walk.pos = app_offsets[group * 32];
  long long at;
  while (walk.step(lane, left > 0, at)) {
    if (left > 0) {
      if (i < end && at < app_capacity) {
        const float2 wk = __ldg(packed + i);
        app_ids[at] = ((uint32_t)ray << kbits) | (uint32_t)__float_as_int(wk.y);
        app_weight[at] = wk.x;
      }
      ++i;
      --left;
    }
  }
}

// rgb_map = sum_j w_j rgb_j (+ 1 - acc), clamp to [0,1]; depth_map = sum w t
// (app/models/gridnerf_sequential.py:493-501).  One thread per ray, ranks in order.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
composite_kernel(const float* __restrict__ app_weight, const int32_t* __restrict__ app_counts,
                 const int32_t* __restrict__ app_offsets, const float* __restrict__ app_rgb, const float* __restrict__ acc, const float* __restrict__ depth,
                 int64_t n_rays, long long app_capacity, int white_bg, float* __restrict__ rgb_map,
                 float* __restrict__ depth_map) {
  const int lane = threadIdx.x & 31;
  const int64_t group = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (group * 32 >= n_rays) return;
  const int64_t ray = group * 32 + lane;
  const bool has_ray = ray < n_rays;
  int left = has_ray ? app_counts[ray] : 0;
  float r = 0.0f, g = 0.0f, b = 0.0f;
  AppGroupWalk walk;
  walk.pos = app_offsets[group * 32];
  long long at;
  while (walk.step(lane, left > 0, at)) {
    if (left > 0) {
      if (at < app_capacity) {
        const float w = __ldg(app_weight + at);
        r = fmaf(w, __ldg(app_rgb + at * 3 + 0), r);
        g = fmaf(w, __ldg(app_rgb + at * 3 + 1), g);
        b = fmaf(w, __ldg(app_rgb + at * 3 + 2), b);
      }
      --left;
    }
  }
  if (has_ray) {
    if (rgb_map) {
      const float bg = white_bg ? (1.0f - acc[ray]) : 0.0f;
      rgb_map[ray * 3 + 0] = fminf(fmaxf(r + bg, 0.0f), 1.0f);
      rgb_map[ray * 3 + 1] = fminf(fmaxf(g + bg, 0.0f), 1.0f);
      rgb_map[ray * 3 + 2] = fminf(fmaxf(b + bg, 0.0f), 1.0f);
    }
    if (depth_map) depth_map[ray] = depth[ray];
  }
}

}  // namespace

int launch_weights_only(const GnrModel* m, const GnrSampleParams& p, int64_t n, char* ws, const GnrWs& L,
                        int64_t max_valid, cudaStream_t st, const float* sigma_rows, const int32_t* rows) {
  unsigned blocks = (unsigned)((n + 31) / 32);
  const bool ext = sigma_rows != nullptr;  // owners' answers read in place through `rows`, packed output
  weights_kernel<<<blocks, 32, 0, st>>>(
      p, m->cfg.distance_scale, m->cfg.ray_weight_thres, (const float*)(ws + L.t_min), (const uint32_t*)(ws + L.words),
      ext ? sigma_rows : (const float*)(ws + L.sigma), (const int32_t*)(ws + L.offsets), n, (long long)max_valid,
      (float*)(ws + L.weight), (float*)(ws + L.acc), (float*)(ws + L.depth), (int32_t*)(ws + L.app_counts),
      ext ? rows : nullptr, ext ? (float2*)(ws + L.sigma) : nullptr);
  return (int)cudaGetLastError();
}

int launch_app_compact(const GnrModel* m, const GnrSampleParams& p, int64_t n, char* ws, const GnrWs& L,
                       int64_t max_valid, int64_t max_app, cudaStream_t st, int packed) {
  int32_t* app_offsets = (int32_t*)(ws + L.app_offsets);
  int e = launch_exclusive_scan((const int32_t*)(ws + L.app_counts), app_offsets, (int32_t*)(ws + L.block_sums), n,
                                (int32_t*)(ws + L.status), GNR_ST_NUM_APP, GNR_ST_OVERFLOW_APP, max_app, st);
  if (e) return e;
  const int64_t groups = (n + 31) / 32;
  unsigned blocks = (unsigned)((groups + kWarpsPerBlock - 1) / kWarpsPerBlock);
  if (packed) {
    expand_app_packed_kernel<<<blocks, kWarpsPerBlock * 32, 0, st>>>(
        (const float2*)(ws + L.sigma), p.kbits, (const int32_t*)(ws + L.offsets),
        (const int32_t*)(ws + L.app_counts), app_offsets, n, (long long)max_valid, (long long)max_app,
        (uint32_t*)(ws + L.app_ids), (float*)(ws + L.app_weight));
    return (int)cudaGetLastError();
  }
  expand_app_kernel<<<blocks, kWarpsPerBlock * 32, 0, st>>>((const float*)(ws + L.weight), (const uint32_t*)(ws + L.words),
                                                           p.words, p.kbits, m->cfg.ray_weight_thres,
                                                           (const int32_t*)(ws + L.offsets),
                                                           (const int32_t*)(ws + L.app_counts), app_offsets, n,
                                                           (long long)max_valid, (long long)max_app,
                                                           (int32_t*)(ws + L.app_index), (uint32_t*)(ws + L.app_ids),
                                                           (float*)(ws + L.app_weight));
  return (int)cudaGetLastError();
}

int launch_composite(const GnrModel* m, int64_t n, int white_bg, char* ws, const GnrWs& L, float* rgb_map,
                     float* depth_map, cudaStream_t st) {
  (void)m;
  const int64_t groups = (n + 31) / 32;
  unsigned blocks = (unsigned)((groups + kWarpsPerBlock - 1) / kWarpsPerBlock);
  long long app_capacity = L.max_app;
  composite_kernel<<<blocks, kWarpsPerBlock * 32, 0, st>>>(
      (const float*)(ws + L.app_weight), (const int32_t*)(ws + L.app_counts), (const int32_t*)(ws + L.app_offsets),
      (const float*)(ws + L.app_rgb), (const float*)(ws + L.acc), (const float*)(ws + L.depth), n, app_capacity,
      white_bg, rgb_map, depth_map);
  return (int)cudaGetLastError();
}

namespace {
__global__ void rgba8_kernel(const float* __restrict__ rgb, long long n, uchar4* __restrict__ out) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float r = rgb[i * 3 + 0] * 255.0f, g = rgb[i * 3 + 1] * 255.0f, b = rgb[i * 3 + 2] * 255.0f;
  out[i] = make_uchar4((unsigned char)__float2uint_rz(fminf(fmaxf(r, 0.0f), 255.0f)),
                       (unsigned char)__float2uint_rz(fminf(fmaxf(g, 0.0f), 255.0f)),
                       (unsigned char)__float2uint_rz(fminf(fmaxf(b, 0.0f), 255.0f)), 255);
}
}  // namespace

extern "C" int gnr_rgba8(const float* rgb, int64_t n, uint8_t* rgba, void* stream) {
  if (!rgb || !rgba || n < 0) {
    gnr_set_error("gnr_rgba8: bad argument");
    return -1;
  }
  if (n == 0) return 0;
  rgba8_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(rgb, (long long)n, reinterpret_cast<uchar4*>(rgba));
  GNR_CUDA_OK(cudaGetLastError());
  return 0;
}
