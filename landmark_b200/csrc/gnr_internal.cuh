// Internal declarations shared by the translation units of libgridnerf_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "gridnerf_b200.h"

#define GNR_MAX_PLANES 9
#define GNR_SM_COUNT_FALLBACK 148

// One plane/line pair in device layout: plane [H][W][C] channel-last, line [L][C];
// C is the padded channel count (multiple of 16, extra channels are zero).
struct GnrPlane {
  const float* plane;
  const float* line;
  int H, W, L, C;
  float fw, fh, fl;  // (float)(W - 1), (H - 1), (L - 1)
  int mat0, mat1, vec;  // coordinate axes: plane x <- xyz[mat0], plane y <- xyz[mat1], line <- xyz[vec]
};

struct GnrMlp {
  // fp32 images for the CUDA-core kernels
  float* basis_raw;      // [app_dim][n_pairs * n_app] as uploaded (source of the appearance lattice)
  float* basis_blocked;  // [4 lanes][36(+pad)][28] blocked basis weights for the gather kernel
  float* w1t;            // [K1p][hidden]  (transposed, K padded)
  float* w2t;            // [hidden][hidden]
  float* w3;             // [3][hidden]
  float* b1;             // [hidden] (zeros if no bias)
  float* b2;
  float* b3;             // [4]
  // tensor-core images (pre-tiled, see gnr_mlp_tc.cu)
  void* tc_image;
  size_t tc_image_bytes;
  int in_dim;   // 150
  int k1_pad;   // in_dim rounded up to 8
  int n_prod;   // sum of padded appearance channels (144)
};

struct GnrProfiler;

struct GnrModel {
  GnrConfig cfg;
  GnrProfiler* prof;  // null unless profiling is enabled
  int device;
  int sm_count;
  GnrPlane den[GNR_MAX_PLANES];
  GnrPlane app[GNR_MAX_PLANES];
  float* den_plane_buf[GNR_MAX_PLANES];
  float* den_line_buf[GNR_MAX_PLANES];
  float* app_plane_buf[GNR_MAX_PLANES];
  float* app_line_buf[GNR_MAX_PLANES];
  size_t plane_bytes[2][GNR_MAX_PLANES];  // current size of every plane / line buffer: an upload of the
  size_t line_bytes[2][GNR_MAX_PLANES];   // same size reuses it (no cudaFree, hence no device-wide sync)
  // projected-feature lattice of the appearance field [gx][gy][gz][32] fp16 (null unless built)
  void* app_lattice;
  size_t app_lattice_bytes;
  int app_lat_dims[3];
  int app_lat_valid;
  // pre-summed density lattice [gx][gy][gz] (null unless built; see gnr_build_density_lattice)
  float* den_lattice;
  size_t den_lattice_bytes;
  int lat_dims[3];
  int lat_valid;  // 0 after a density plane or line was uploaded: the lattice must be rebuilt before the next launch
  // occupancy bits
  uint32_t* alpha_bits;
  uint32_t* alpha_coarse;  // one bit per 4x4x4 block of mask cells (see coarse_bits_kernel)
  uint32_t* alpha_full;    // one bit per block: every cell of the block and of its +1 border is set
  int aD, aH, aW;
  float a_lo[3], a_inv[3];
  GnrMlp mlp;
  int debug_expire_wait;  // test hook (gnr_debug_wait): make one bounded wait of the tensor-core kernels run out
  int debug_wait_limit;   // polls a bounded wait may take; 0 = the default
  int32_t* route_scratch;  // per-CTA block counts and start rows of gnr_route_blocks
  size_t route_scratch_bytes;
  long long* debug_prof;  // device buffer of phase cycle sums (gnr_debug_phase_cycles), null when off
  // hull sampler tables (sampling_mode 1)
  float* hull_near_term;
  float* hull_u;
  int hull_samples;
  // staging for gnr_render_host
  void* host_ws;
  size_t host_ws_bytes;
  float* host_rays;
  float* host_rgb;
  float* host_depth;
  int64_t host_chunk;
  int32_t* host_status;  // pinned
  int64_t host_status_slots;
  cudaStream_t host_streams[2];
  cudaEvent_t host_events[2];
};

// Scalar parameters every sampling-dependent kernel needs (passed by value).
struct GnrSampleParams {
  float lo[3], hi[3], inv[3];
  float near_t, far_t, step;
  float a_lo[3], a_inv[3];
  float a_thres;
  int aD, aH, aW;
  int has_mask;
  const uint32_t* a_bits;
  const uint32_t* a_coarse;  // null, or 1 bit per 4x4x4 block: set if any cell of the block or of its +1 border is set
  const uint32_t* a_full;    // null, or 1 bit per 4x4x4 block: every cell of the block and its +1 border is set
  int cD, cH, cW;
  int S, words, kbits;
  int mode;                 // 0 dense sampler, 1 hull sampler
  const float* hull_a;      // near * (1 - u[k])
  const float* hull_u;      // u[k]
};

// Workspace layout (byte offsets), identical for every stage call with the same arguments.
struct GnrWs {
  size_t status, t_min, words, counts, offsets, block_sums, ids, sigma_feat, sigma, weight, acc, depth,
      app_counts, app_offsets, app_index, app_ids, app_weight, app_feat, app_rgb, app_prod, total;
  size_t app_prod_image;  // bytes of one fp16 product image (hi), 0 if the tensor-core path is off
  int app_prod_tile;      // bytes of one 128-sample tile of that image
  int feat_stride;  // floats per appearance feature row (app_dim rounded up to 4)
  long long max_valid, max_app;  // capacities of the two compacted lists
  long long n_rays;
};

// Where a per-sample kernel finds item i: either through the chunk's compacted lists
// (ids[index ? index[i] : i] -> ray, sample -> position recomputed from the ray) or, in point
// mode, from explicit arrays of normalised positions / view directions.
struct GnrCoords {
  const float* rays;
  const float* t_min;
  const uint32_t* ids;
  const int32_t* index;       // optional indirection (appearance list -> valid list)
  const float* xyz_direct;    // [n][3] normalised positions (point mode)
  const float* view_direct;   // [n][3] view directions (point mode)
  int point_stride;           // floats from one point's row to the next in xyz_direct / view_direct (3 when each is its own array)
  // List mode at a block owner: the position, computed in the GLOBAL box of the sampler, is then expressed in the
  // coordinates of block (blk_bx, blk_by) of a blk_px x blk_py division (blk_px == 0: no blocks).
  int blk_px, blk_py, blk_bx, blk_by;
  float blk_pw, blk_ph;       // 2 / px, 2 / py as fp32
  const int32_t* total_ptr;   // device count of items, or null ...
  long long total_direct;     // ... then this host count
  long long capacity;
};

void gnr_set_error(const char* fmt, ...);
GnrWs gnr_ws_layout(const GnrModel* m, int64_t n_rays, int S, int64_t max_valid, int64_t max_app);
GnrSampleParams gnr_sample_params(const GnrModel* m, int S);
// What every launch of the sampler needs from the model, checked on the host before anything is
// enqueued: with sampling_mode 1 the hull tables must have been uploaded for exactly S samples.
int gnr_check_sampler(const GnrModel* m, int S);
int gnr_check_lattice(const GnrModel* m);  // refuses a lattice that is older than the density planes
int gnr_check_chunk(const GnrModel* m, int64_t n_rays, int S, int64_t max_valid, int64_t max_app,
                    const void* ws, size_t ws_bytes);

// launchers (each enqueues on `st`, returns cudaGetLastError as int)
int launch_sample_mask(const GnrModel* m, const GnrSampleParams& p, const float* rays, int64_t n, char* ws,
                       const GnrWs& L, cudaStream_t st);
// with_ids == 0: offsets only (the compacted id list is needed by the list-based density kernel and the stage API)
int launch_sample_compact(const GnrModel* m, const GnrSampleParams& p, int64_t n, char* ws, const GnrWs& L,
                          int64_t max_valid, int with_ids, cudaStream_t st);
int launch_build_lattice(const GnrModel* m, float* V, cudaStream_t st);
int launch_build_app_lattice(const GnrModel* m, void* V, cudaStream_t st);
int gnr_app_lattice_dims(const GnrModel* m, int* dims);
int gnr_lattice_dims(const GnrModel* m, int* dims);  // grid of the density field if it has the standard VM3 layout, else -1
GnrCoords gnr_coords_valid(const float* rays, char* ws, const GnrWs& L);
GnrCoords gnr_coords_app(const float* rays, char* ws, const GnrWs& L);
int launch_density(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, float* sigma_feat, float* sigma,
                   cudaStream_t st);
// (`sigma_rows` + `rows`: sigma of list entry i is sigma_rows[rows[i]], read in place; the output is then the packed
// form launch_app_compact(..., packed = 1) reads)
int launch_weights_only(const GnrModel* m, const GnrSampleParams& p, int64_t n, char* ws, const GnrWs& L,
                        int64_t max_valid, cudaStream_t st, const float* sigma_rows = nullptr, const int32_t* rows = nullptr);
// (`packed`: the march ran with list_only)
int launch_app_compact(const GnrModel* m, const GnrSampleParams& p, int64_t n, char* ws, const GnrWs& L,
                       int64_t max_valid, int64_t max_app, cudaStream_t st, int packed = 0);
// Fused density gather + transmittance scan + early termination, one warp per ray.
// (`list_only`: instead of one weight per valid sample, write only the samples above the appearance threshold, packed
// at the front of every ray's range as 8-byte (weight, sample number) pairs in the sigma + weight arrays, which lie
// back to back in the workspace; what
// launch_app_compact(..., packed = 1) reads)
int launch_march(const GnrModel* m, const GnrSampleParams& p, const float* rays, int64_t n, char* ws, const GnrWs& L,
                 cudaStream_t st, int list_only = 0);
int launch_app_gather(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, int feat_stride, float* feat,
                      cudaStream_t st);
int launch_app_products(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, unsigned char* prod_hi,
                        unsigned char* prod_lo, int tile_bytes, int terms, cudaStream_t st);
// gather + basis + MLP in one kernel (gnr_app_fused.cu): 1 if this model can run it
int gnr_app_fusable(const GnrModel* m);
// the same work with dedicated gather warps feeding the MLP warps through tensor memory (gnr_app_stream.cu)
int launch_app_mlp_stream(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, float* rgb, int32_t* status,
                          cudaStream_t st);
// (`features` non-null: MLP alone on given projected features [n][feat_stride] and c.view_direct)
int launch_app_mlp_fused(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, float* rgb, int32_t* status,
                         cudaStream_t st, const float* features = nullptr, int feat_stride = 0,
                         const void* parts_h = nullptr, int n_parts = 0, int64_t part_stride_rows = 0);
// partial projection of a channel slice at explicit points, fp16 rows of 32 (gnr_app_slice.cu), and the fp32 sum of such parts
int launch_app_slice_project(const GnrModel* m, const float* xyz, int stride, int64_t n, void* features_h, int32_t* status,
                             cudaStream_t st);
int launch_sum_partials(const void* parts_h, int n_parts, int64_t rows, int64_t part_stride_rows, int n_out, int out_stride,
                        float* out, cudaStream_t st);
void gnr_fused_k1_order(int* map);  // K order of the fused kernel's layer-1 operand (160 entries)
int gnr_tc_basis_fused(const GnrModel* m);  // 1 if the tensor-core path also runs the basis projection
int gnr_tc_tile_bytes(const GnrModel* m);   // bytes of one 128-sample product tile (products + the view group)
// (`mode` 0: rows of block-local points; 1: points + view directions; 2: 32-bit ids, (ray_base + ray) << kbits | sample)
int launch_route_blocks(GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, int px, int py, int mode, float* send,
                        int32_t* dest, int32_t* counts, int32_t* block_of, cudaStream_t st, uint32_t ray_base = 0);
int launch_positions(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, float* xyz, int32_t* ray_index,
                     cudaStream_t st);
int launch_mlp_simt(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, int feat_stride, const float* feat,
                    float* rgb, cudaStream_t st);
// feat_in: features for the non-fused variant; feat_out: optional copy of the projected features
// (fused variant); prod_*: product tiles (fused variant); status: 8-word block for the wait flag.
int launch_mlp_tc(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, int feat_stride, const float* feat_in,
                  float* feat_out, const unsigned char* prod_hi, const unsigned char* prod_lo, int tile_bytes, float* rgb,
                  int32_t* status, int force_unfused, cudaStream_t st, int basis_only = 0);
int launch_composite(const GnrModel* m, int64_t n, int white_bg, char* ws, const GnrWs& L, float* rgb_map,
                     float* depth_map, cudaStream_t st);
int launch_exclusive_scan(const int32_t* counts, int32_t* offsets, int32_t* block_sums, int64_t n,
                          int32_t* status, int total_slot, int overflow_slot, int64_t capacity,
                          cudaStream_t st);
int gnr_mlp_tc_prepare(GnrModel* m, const float* basis_w, const float* w1, const float* w2, const float* w3,
                       cudaStream_t st);

#define GNR_CUDA_OK(expr)                                                              \
  do {                                                                                 \
    cudaError_t _e = (expr);                                                           \
    if (_e != cudaSuccess) {                                                           \
      gnr_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return -2;                                                                       \
    }                                                                                  \
  } while (0)

// ---- device helpers shared by the sampling-dependent kernels ---------------------------------
// Every operation is individually rounded (no FMA contraction): these reproduce the values
// torch computes with separate elementwise kernels.
// Distance of sample k along a ray.  Dense sampler: t_min + stepSize * k with the ray's slab
// entry t_min; hull sampler: near * (1 - u_k) + far * u_k with the ray's own far
// (app/models/gridnerf_sequential.py:268-273 and :303-304).  `ray_param` is t_min resp. far.
__device__ __forceinline__ float gnr_sample_t(const GnrSampleParams& p, float ray_param, int k) {
  if (p.mode == 0) return __fadd_rn(ray_param, __fmul_rn(p.step, (float)k));
  return __fadd_rn(__ldg(p.hull_a + k), __fmul_rn(ray_param, __ldg(p.hull_u + k)));
}
__device__ __forceinline__ float gnr_point(float o, float d, float t) { return __fadd_rn(o, __fmul_rn(d, t)); }
__device__ __forceinline__ float gnr_normalize(float p, float lo, float inv) {
  return __fsub_rn(__fmul_rn(__fsub_rn(p, lo), inv), 1.0f);
}
