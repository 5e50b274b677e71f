// Block routing for a field cut into Px x Py blocks that live on different GPUs.
//
// assign_blocks_to_samples (app/models/gridnerf_parallel.py:279-338; the reference's kernel version is
// dist_render/kernel/cuda_kernel/sampleray_gridsample/compute_assign_blocks_to_samples_norm_cuda_kernel.cu:19-74)
// gives every sample the block that holds it and its coordinates inside that block.  Here the same
// arithmetic runs on the entries of a chunk's valid list or appearance list and, in the same pass,
// groups the samples by owning block: the output is the send buffer of an all-to-all (block-local
// points, block 0's first) plus, per list entry, the row it went to, and the per-block counts.
//
// Three launches, no atomics on global memory, no host synchronisation:
//   count:   every CTA owns a contiguous share of the list and counts its entries per block;
//   scan:    one CTA turns the [CTA][block] counts into start rows (block-major, CTA-minor);
//   scatter: every CTA walks its share again, in order, and writes each entry at the next free row of
//            its block's range.
// The order inside a block's range is therefore the list order (a stable partition), which is what a
// per-block `nonzero` gives, so results do not depend on how the CTAs were scheduled.
//
// Every floating-point step is a single rounded fp32 operation in torch's order (true division, as
// the CPU path of torch divides), so block indices and block-local coordinates have the bits of the
// reference's own method.  One intended difference: a sample with x or y exactly 1 belongs to the
// last block here (the reference gives it an index past the last block).
#include "gnr_gather.cuh"

namespace {

constexpr int kRouteBlock = 256;
constexpr int kRouteWarps = kRouteBlock / 32;
constexpr int kMaxBlocks = 32;  // blocks (ranks) per field

struct BlockGrid {
  int px, py;
  float pw, ph;  // 2 / px, 2 / py as fp32 (what a python float becomes next to an fp32 tensor)
};

// block index and block-local x, y of a normalised position
__device__ __forceinline__ int assign_block(const BlockGrid& g, float x, float y, float& lx, float& ly) {
  const float u = __fdiv_rn(__fadd_rn(x, 1.0f), g.pw), v = __fdiv_rn(__fadd_rn(y, 1.0f), g.ph);
  const float bx = fminf(fmaxf(floorf(u), 0.0f), (float)(g.px - 1)), by = fminf(fmaxf(floorf(v), 0.0f), (float)(g.py - 1));
  block_local(bx, by, g.pw, g.ph, x, y, lx, ly);
  return (int)bx * g.py + (int)by;
}

// contiguous share of [0, total) for this CTA, a multiple of the block size long
__device__ __forceinline__ void route_range(long long total, long long& beg, long long& end) {
  const long long steps = (total + kRouteBlock - 1) / kRouteBlock;
  const long long per = (steps + gridDim.x - 1) / gridDim.x;
  beg = min(total, (long long)blockIdx.x * per * kRouteBlock);
  end = min(total, beg + per * kRouteBlock);
}

__global__ void __launch_bounds__(kRouteBlock)
route_count_kernel(GnrSampleParams p, GnrCoords crd, BlockGrid g, int n_blocks, int32_t* __restrict__ cta_counts) {
  __shared__ int s_cnt[kMaxBlocks];
  if (threadIdx.x < kMaxBlocks) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  const long long total = coords_total(crd);
  long long beg, end;
  route_range(total, beg, end);
  for (long long base = beg; base < end; base += kRouteBlock) {
    const long long i = base + threadIdx.x;
    int b = -1;
    if (i < end) {
      float x, y, z, lx, ly;
      sample_xyz(p, crd, i, x, y, z);
      b = assign_block(g, x, y, lx, ly);
    }
    // one shared-memory add per (warp, block) instead of one per sample
    const uint32_t same = __match_any_sync(0xffffffffu, b);
    if (b >= 0 && (same & ((1u << (threadIdx.x & 31)) - 1u)) == 0u) atomicAdd(&s_cnt[b], __popc(same));
  }
  __syncthreads();
  if (threadIdx.x < n_blocks) cta_counts[(size_t)blockIdx.x * kMaxBlocks + threadIdx.x] = s_cnt[threadIdx.x];
}

// cta_counts[cta][block] -> cta_base[cta][block] (start row of that CTA's entries of that block) and counts[block]
__global__ void __launch_bounds__(kMaxBlocks) route_scan_kernel(const int32_t* __restrict__ cta_counts, int n_ctas, int n_blocks,
                                                                 int32_t* __restrict__ cta_base, int32_t* __restrict__ counts) {
  __shared__ int s_total[kMaxBlocks];
  const int b = threadIdx.x;
  int sum = 0;
  if (b < n_blocks) {
    for (int c = 0; c < n_ctas; ++c) sum += cta_counts[(size_t)c * kMaxBlocks + b];
    counts[b] = sum;
  }
  s_total[b] = b < n_blocks ? sum : 0;
  __syncthreads();
  if (b < n_blocks) {
    int start = 0;
    for (int k = 0; k < b; ++k) start += s_total[k];
    for (int c = 0; c < n_ctas; ++c) {
      cta_base[(size_t)c * kMaxBlocks + b] = start;
      start += cta_counts[(size_t)c * kMaxBlocks + b];
    }
  }
}

// MODE 0: rows of (block-local x, y, z); 1: the same plus the view direction; 2: one 32-bit id per row,
// (ray_base + ray) << kbits | sample: the owner recomputes the position from the ray itself (it holds the rays of
// every rank of the chunk, rank r's first ray at its ray_base), a third of the bytes on the wire for a valid sample
// and a sixth for an appearance sample.
template <int MODE>
__global__ void __launch_bounds__(kRouteBlock)
route_scatter_kernel(GnrSampleParams p, GnrCoords crd, BlockGrid g, int n_blocks, const int32_t* __restrict__ cta_base,
                     float* __restrict__ send, int32_t* __restrict__ dest, int32_t* __restrict__ block_of, uint32_t ray_base) {
  constexpr bool WITH_VIEW = MODE == 1;
  __shared__ int s_run[kMaxBlocks];                 // next free row of every block for this CTA
  __shared__ int s_warp[kRouteWarps][kMaxBlocks];   // entries of a block per warp in the current step
  if (threadIdx.x < kMaxBlocks)
    s_run[threadIdx.x] = threadIdx.x < n_blocks ? cta_base[(size_t)blockIdx.x * kMaxBlocks + threadIdx.x] : 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int kStride = WITH_VIEW ? 6 : 3;
  const long long total = coords_total(crd);
  long long beg, end;
  route_range(total, beg, end);
  for (long long base = beg; base < end; base += kRouteBlock) {
    if (threadIdx.x < kRouteWarps * kMaxBlocks / 8) {
#pragma unroll
      for (int k = 0; k < 8; ++k) (&s_warp[0][0])[threadIdx.x * 8 + k] = 0;
    }
    __syncthreads();
    const long long i = base + threadIdx.x;
    int b = -1;
    float lx = 0.0f, ly = 0.0f, z = 0.0f, view[3] = {0.0f, 0.0f, 0.0f};
    if (i < end) {
      float x, y;
      sample_xyz(p, crd, i, x, y, z, WITH_VIEW ? view : nullptr);
      b = assign_block(g, x, y, lx, ly);
    }
    const uint32_t same = __match_any_sync(0xffffffffu, b);
    const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
    if (b >= 0 && rank_in_warp == 0) s_warp[warp][b] = __popc(same);
    __syncthreads();
    if (b >= 0) {
      int row = s_run[b] + rank_in_warp;
      for (int w = 0; w < warp; ++w) row += s_warp[w][b];
      if (MODE == 2) {
        const uint32_t id = __ldg(crd.ids + i);
        reinterpret_cast<uint32_t*>(send)[row] = id + (ray_base << p.kbits);
      } else {
        float* out = send + (size_t)row * kStride;
        out[0] = lx;
        out[1] = ly;
        out[2] = z;
        if (WITH_VIEW) {
          out[3] = view[0];
          out[4] = view[1];
          out[5] = view[2];
        }
      }
      dest[i] = row;
      if (block_of) block_of[i] = b;
    }
    __syncthreads();
    if (threadIdx.x < n_blocks) {
      int add = 0;
#pragma unroll
      for (int w = 0; w < kRouteWarps; ++w) add += s_warp[w][threadIdx.x];
      s_run[threadIdx.x] += add;
    }
    __syncthreads();
  }
}

}  // namespace

int launch_route_blocks(GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, int px, int py, int mode, float* send,
                        int32_t* dest, int32_t* counts, int32_t* block_of, cudaStream_t st, uint32_t ray_base) {
  const int n_blocks = px * py;
  if (px < 1 || py < 1 || n_blocks > kMaxBlocks) {
    gnr_set_error("block routing supports 1..%d blocks (got %d x %d)", kMaxBlocks, px, py);
    return -1;
  }
  const int n_ctas = m->sm_count * 4;
  const size_t need = (size_t)n_ctas * kMaxBlocks * 2 * sizeof(int32_t);
  if (!m->route_scratch || m->route_scratch_bytes < need) {
    if (m->route_scratch) {
      cudaDeviceSynchronize();
      cudaFree(m->route_scratch);
    }
    m->route_scratch = nullptr;
    m->route_scratch_bytes = 0;
    GNR_CUDA_OK(cudaMalloc(&m->route_scratch, need));
    m->route_scratch_bytes = need;
  }
  int32_t* cta_counts = m->route_scratch;
  int32_t* cta_base = cta_counts + (size_t)n_ctas * kMaxBlocks;
  BlockGrid g;
  g.px = px;
  g.py = py;
  g.pw = (float)(2.0 / px);
  g.ph = (float)(2.0 / py);
  route_count_kernel<<<n_ctas, kRouteBlock, 0, st>>>(p, c, g, n_blocks, cta_counts);
  route_scan_kernel<<<1, kMaxBlocks, 0, st>>>(cta_counts, n_ctas, n_blocks, cta_base, counts);
  if (mode == 2)
    route_scatter_kernel<2><<<n_ctas, kRouteBlock, 0, st>>>(p, c, g, n_blocks, cta_base, send, dest, block_of, ray_base);
  else if (mode == 1)
    route_scatter_kernel<1><<<n_ctas, kRouteBlock, 0, st>>>(p, c, g, n_blocks, cta_base, send, dest, block_of, 0u);
  else
    route_scatter_kernel<0><<<n_ctas, kRouteBlock, 0, st>>>(p, c, g, n_blocks, cta_base, send, dest, block_of, 0u);
  return (int)cudaGetLastError();
}
