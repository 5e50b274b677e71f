/*
 * gridnerf_b200 -- C ABI of the B200 (sm_100a) GridNeRF render path.
 *
 * This is the boundary a host binds instead of the reference's per-chunk ``_forward``
 * callable (dist_render/ddp_infer/inferer_impl.py:36,60-61,107-119) and instead of the
 * pybind kernel modules that its kernel-fusion path chains
 * (dist_render/kernel/cuda_render_extend.py:4-22,350-526).
 *
 * Conventions
 *  - plain C types only; every pointer is a DEVICE pointer unless its name ends in ``_h``;
 *  - every call that enqueues work takes the CUDA stream (``void*`` = ``cudaStream_t``) and
 *    never synchronises it, except the ``*_host`` calls, which return finished host buffers;
 *  - return value 0 = ok, negative = error detected on the host before anything was
 *    enqueued (``gnr_last_error`` gives the text).  Conditions only the device can see
 *    (a compacted list larger than its capacity) are written into the 8-word status block
 *    at the start of the workspace and read back with ``gnr_read_status``;
 *  - nothing here falls back to the CPU.
 */
#ifndef GRIDNERF_B200_H
#define GRIDNERF_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct GnrModel GnrModel;

/* Scalar description of one field.  The float members are passed as the exact fp32 values
 * the reference computes with torch (update_stepSize, app/models/gridnerf_sequential.py:149-164;
 * AlphaGridMask.__init__, app/models/alpha_mask.py:16-26) so that sampling is bit-exact. */
typedef struct GnrConfig {
  float aabb[6];            /* min x,y,z then max x,y,z                        (:91)      */
  float inv_aabb_size[3];   /* 2 / (max - min)                                 (:159)     */
  int32_t grid[3];          /* gridSize x,y,z                                  (:160)     */
  float near_t, far_t;      /* near_far                                        (:101)     */
  float step_size;          /* mean(units) * step_ratio                        (:162)     */
  float distance_scale;     /*                                                  (:97)      */
  float density_shift;      /*                                                  (:95)      */
  int32_t density_act;      /* 0 = softplus(x + shift), 1 = relu(x)            (:386-399) */
  float ray_weight_thres;   /* rayMarch_weight_thres: app_mask = w > thres     (:479)     */
  float alpha_filter_thres; /* alpha_mask_filter_thre                          (:462)     */
  int32_t n_pairs;          /* plane/line pairs per kind = ndims * len(resMode) (:106-110) */
  int32_t n_density;        /* channels of every density plane/line            (:88)      */
  int32_t n_app;            /* channels of every appearance plane/line         (:89)      */
  int32_t app_dim;          /* basis_mat output width (27)                     (:678)     */
  int32_t fea_pe, view_pe;  /* positional-encoding octaves (mlp_render_fea.py:20-27)      */
  int32_t hidden;           /* featureC (128)                                             */
  int32_t has_bias;         /* bias_enable                                                */
  int32_t mlp_mode;         /* 0 = fp32 CUDA-core MLP, 1 = tcgen05 split-precision MLP (fp32-grade),
                               2 = tcgen05 MLP with single fp16 operands, fp32 accumulate (fast) */
  int32_t sampling_mode;    /* 0 = sample_ray (:244-281), 1 = sample_ray_within_hull (:283-319,
                               args.sampling_opt); mode 1 needs gnr_upload_hull_tables             */
  float ert_transmittance;  /* early ray termination of the fused density + weights pass: a ray stops
                               taking density samples once its transmittance falls below this value
                               (its rgb then differs from the unterminated result by less than the
                               value).  0 = never terminate (exact); negative = use the separate
                               density and weights kernels instead of the fused pass.             */
  int32_t app_storage;      /* 0 = appearance planes and lines held as fp32; 1 = held as fp16 (half the
                               gather traffic; the products they feed are rounded to fp16 for the
                               tensor cores anyway).  The reference's half_precision_param does this to
                               the planes of its tensor-parallel model
                               (dist_render/ddp_infer/inferer_impl.py:263-267; there the density planes
                               too, here they stay fp32).  1 needs mlp_mode 2 and 33..48 appearance
                               channels. */
  int32_t den_storage;      /* the same for the density planes and lines (the other half of the
                               reference's half_precision_param); any mlp_mode; 16 (padded) density
                               channels.  Sample sets do not depend on it; rgb moves by a few 1e-6. */
  int32_t unfused_appearance; /* 0 = gnr_render_chunk runs appearance gather, basis projection and MLP as ONE
                               kernel whenever the model allows it (mlp_mode 2, app_storage 1, 48 padded
                               appearance channels, at most 160 products per sample): three groups of warps
                               each gather and then run the MLP of their own tile, the three tiles sharing two
                               accumulators in tensor memory; 1 = always the separate gather and MLP kernels
                               (what the stage-wise entries run); 2 = the one-kernel form with dedicated gather
                               warps feeding the MLP warps through tensor memory; 3 = the one-kernel form with
                               two groups, one accumulator each (2 and 3: same results, kept as measured
                               alternatives).                                                             */
  int32_t reserved[3];
} GnrConfig;

/* Indices into the 8 x int32 status block (first 32 bytes of every workspace). */
enum {
  GNR_ST_OVERFLOW_VALID = 0, /* 1 if #valid samples exceeded max_valid                    */
  GNR_ST_OVERFLOW_APP = 1,   /* 1 if #appearance samples exceeded max_app                 */
  GNR_ST_NUM_VALID = 2,      /* #samples passing the box + occupancy test                 */
  GNR_ST_NUM_APP = 3,        /* #samples with weight > ray_weight_thres                   */
  GNR_ST_WAIT_EXPIRED = 4,   /* a bounded device-side wait gave up (tensor-core MLP)      */
  GNR_ST_NUM_DENSITY = 5,    /* #samples whose density was evaluated (fused pass; < NUM_VALID
                                when early ray termination is on)                          */
  GNR_ST_WORDS = 8
};

const char* gnr_last_error(void);
int gnr_version(void);

/* Model lifetime.  Replaces GridNeRF(**kwargs) + .load(ckpt)
 * (dist_render/ddp_infer/inferer_impl.py:134-142).  ``device`` is the CUDA ordinal. */
int gnr_create(const GnrConfig* cfg_h, int device, GnrModel** out_h);
int gnr_destroy(GnrModel* m);

/* Parameter upload: the source is the reference's checkpoint layout, converted on the
 * device to this library's layout (channel-last planes ``[H][W][C]``, lines ``[L][C]``,
 * channels zero-padded to a multiple of 16).  kind 0 = density, 1 = appearance; ``idx`` is
 * the position in the reference's ParameterList (plane ``idx`` belongs to dimension
 * ``idx / len(resMode)``).  ``axis_x``/``axis_y`` are matMode[dim] (the xyz components that
 * index the plane's W and H) and ``axis`` is vecMode[dim].
 * Replaces load_state_dict of density_plane/app_plane ``[1,C,H,W]`` and
 * density_line/app_line ``[1,C,L,1]`` (app/models/gridnerf_sequential.py:106-107,676-677,703-718). */
int gnr_upload_plane(GnrModel* m, int kind, int idx, const float* src_chw, int C, int H, int W, int axis_x,
                     int axis_y, void* stream);
int gnr_upload_line(GnrModel* m, int kind, int idx, const float* src_cl, int C, int L, int axis, void* stream);
/* Occupancy volume ``[D][H][W]`` of 0/1 bytes, bit-packed on the device; ``aabb_h`` and
 * ``inv_size_h`` are AlphaGridMask.aabb and .invgridSize (app/models/alpha_mask.py:20-22).
 * Passing ``vol = NULL`` removes the mask (alphaMask is None, gridnerf_sequential.py:460). */
int gnr_upload_alpha_mask(GnrModel* m, const uint8_t* vol, int D, int H, int W, const float* aabb_h,
                          const float* inv_size_h, void* stream);
/* basis_mat.weight ``[app_dim][sum n_app]`` and renderModule.mlp.{0,2,4}.{weight,bias}
 * (row-major ``[out][in]``; bias pointers may be NULL).  app/models/mlp_render_fea.py:29-42. */
int gnr_upload_mlp(GnrModel* m, const float* basis_w, const float* w1, const float* b1, const float* w2,
                   const float* b2, const float* w3, const float* b3, void* stream);

/* Optional pre-summed density lattice.  For the standard three-pair layout on one grid,
 * compute_densityfeature (app/models/gridnerf_sequential.py:779-827: per pair, bilinear plane sample x
 * linear line sample, summed over channels and pairs) is exactly the trilinear interpolation of one
 * scalar per grid point, V[x][y][z] = sum over pairs and channels of plane texel x line entry.  With
 * ``enable`` != 0 this builds V on the device from the density planes and lines uploaded so far
 * (4 bytes x grid points, e.g. 4.3 GB for 2048x2048x256; each value is the correctly rounded sum) and
 * every later density evaluation of the model (gnr_render_chunk, gnr_march, gnr_density,
 * gnr_density_points) reads 8 scalars per sample from it instead of 18 texels of 16 channels; the
 * feature differs from the plane/line evaluation only by floating-point summation order.  Uploading
 * a density plane or line afterwards makes the lattice stale: launches are refused until it is
 * rebuilt (same size: no allocation, stream-ordered).  ``enable`` == 0 frees it.  Needs n_pairs == 3
 * with the planes (x,y), (x,z), (y,z) of one grid; refused otherwise. */
int gnr_build_density_lattice(GnrModel* m, int enable, void* stream);

/* Optional projected-feature lattice of the appearance field ("baked" appearance).  compute_appfeature
 * (app/models/gridnerf_sequential.py:829-871) is basis_mat applied to the plane x line products, and every
 * product is trilinear in the position, so the 27 projected features are the trilinear interpolation of
 * their values at the eight surrounding grid points.  With ``enable`` != 0 this builds those values on the
 * device (32 fp16 channels = 64 bytes per grid point: 69 GB for 2048x2048x256, refused if the device has
 * not that much free) from the appearance planes, lines and basis matrix uploaded so far, and
 * gnr_render_chunk / gnr_appearance_points then run the one-kernel appearance path without a plane
 * gather and without the projection GEMM: a sample reads 8 x 64 bytes.  Against the plane path the
 * features carry one fp16 rounding per lattice value instead of one per product.  An upload of an
 * appearance plane or line, or of the MLP, makes the lattice stale (launches refused until rebuilt).
 * Needs mlp_mode 2, three pairs in the standard layout, 33..48 appearance channels.  A trade of memory
 * for time, off by default; the stage-wise entries keep reading the planes. */
int gnr_build_appearance_lattice(GnrModel* m, int enable, void* stream);

/* Tables of the hull sampler for ``n_samples`` (= n_importance) samples per ray:
 * ``u[k] = torch.linspace(0, 1, n_samples)[k]`` and ``near_term[k] = near * (1.0 - u[k])``, both
 * evaluated by torch on the CPU so that ``z = near_term[k] + far * u[k]`` has the reference's bits
 * (app/models/gridnerf_sequential.py:303-304).  Device pointers; copied. */
int gnr_upload_hull_tables(GnrModel* m, int n_samples, const float* near_term, const float* u, void* stream);

/* Ray generation from a pose.  Replaces generate_rays (dist_render/dataset/utils.py:92-113):
 * ``dir_x[W]`` and ``dir_y[H]`` are the two torch.arange tables of
 * get_ray_directions_blender_faster (:57-70); ``pose_h`` is the row-major ``[3][4]`` c2w.
 * Ray ``r`` of the output is pixel ``pixel_ids[r]`` (row-major y*W+x), or pixel
 * ``first_pixel + r`` if ``pixel_ids`` is NULL.  Output ``rays[n][6]`` = origin, direction. */
int gnr_generate_rays(const float* pose_h, const float* dir_x, const float* dir_y, int H, int W,
                      const int32_t* pixel_ids, int64_t first_pixel, int64_t n, float* rays, void* stream);

/* gnr_generate_rays with the pose (12 floats, row-major [3][4]) in DEVICE memory, read when the
 * kernel runs: a frame captured as a CUDA graph is replayed for a new pose by rewriting the pose
 * buffer (the role of the per-frame pose broadcast, dist_render/ddp_infer/nerf_inferer.py:150-171). */
int gnr_generate_rays_dev(const float* pose_dev, const float* dir_x, const float* dir_y, int H, int W,
                          const int32_t* pixel_ids, int64_t first_pixel, int64_t n, float* rays, void* stream);

/* Frame post-process on the device: ``out[i] = (uint8)(rgb[i] * 255)`` (truncation, what
 * ``.byte()`` does) with alpha 255, i.e. the ``result * 255`` / ``torch.cat(..., 255)`` / ``.byte()``
 * steps of model_infer_postprocess (dist_render/ddp_infer/nerf_inferer.py:366-370).
 * ``rgb[n][3]`` fp32 -> ``rgba[n][4]`` uint8. */
int gnr_rgba8(const float* rgb, int64_t n, uint8_t* rgba, void* stream);

/* Scratch memory for one chunk.  The caller allocates ``bytes`` (256-byte aligned) and
 * passes it to the calls below; contents carry no state between chunks. */
int gnr_workspace_bytes(const GnrModel* m, int64_t n_rays, int n_samples, int64_t max_valid,
                        int64_t max_app, size_t* bytes_h);

/* The whole per-chunk forward: GridBaseSequential.forward, dense-sampling branch
 * (app/models/gridnerf_sequential.py:448-504) = sample_ray (:244-281) + alphaMask filter
 * (:460-465) + compute_densityfeature (:779-827) + feature2density (:386-399) + raw2alpha
 * (app/tools/utils.py:51-64) + compute_appfeature (:829-871) + MLPRender_Fea.forward
 * (app/models/mlp_render_fea.py:44-68) + compositing (:493-501).
 * ``rays[n][6]`` -> ``rgb_map[n][3]``, ``depth_map[n]`` (either output may be NULL). */
int gnr_render_chunk(GnrModel* m, const float* rays, int64_t n_rays, int n_samples, int white_bg,
                     void* workspace, size_t workspace_bytes, int64_t max_valid, int64_t max_app,
                     float* rgb_map, float* depth_map, void* stream);

/* Same forward with HOST buffers: copies ``rays_h`` to the device in chunks of
 * ``chunk_rays``, renders, copies rgb/depth back, synchronises, and returns the status block.
 * This is the renderer_fn chunk loop (dist_render/ddp_infer/inferer_impl.py:95-120) with its
 * host<->device traffic included.  ``rays_h``/``rgb_h``/``depth_h`` should be pinned. */
int gnr_render_host(GnrModel* m, const float* rays_h, int64_t n_rays, int n_samples, int white_bg,
                    int64_t chunk_rays, int64_t max_valid, int64_t max_app, float* rgb_h, float* depth_h,
                    int32_t* status_h);

/* ---- stage-wise entries (each kernel is parity-testable alone) ---------------------------- */

/* Stage 1: sample_ray + alphaMask filter + compaction.  Outputs (any may be NULL except
 * inside the workspace, where they are always produced): per-ray ``t_min[n]``, per-ray valid
 * ``counts[n]``, exclusive ``offsets[n+1]``, the validity bit words ``mask_words[n][ceil(S/32)]``
 * and the compacted ``ids`` (ray << kbits | sample, kbits = gnr_sample_bits(S)) in the order
 * of ``xyz_sampled[ray_valid]`` (ray-major).  gridnerf_sequential.py:244-281,460-465. */
int gnr_sample(GnrModel* m, const float* rays, int64_t n_rays, int n_samples, void* workspace,
               size_t workspace_bytes, int64_t max_valid, float* t_min, int32_t* counts, int32_t* offsets,
               uint32_t* mask_words, uint32_t* ids, void* stream);
int gnr_sample_bits(int n_samples);

/* Stage 1 again, for callers that must not allocate.  (This entry has no counterpart in the
 * reference.)  The frame loop of an online renderer is such a caller: a cudaMalloc there
 * synchronises the whole device and stalls the other pipeline stages' streams, and a host
 * that has given all of its device memory to the field's planes has nothing left to hand out
 * as a workspace.  gnr_sample_static therefore takes no workspace: its scratch (the validity
 * bit words and the scan's block sums) lives in one fixed array of
 * GNR_SAMPLE_STATIC_SCRATCH_BYTES inside the library, which every GPU that loads the library
 * holds until the process exits.  The call allocates and frees nothing.
 *
 *  - Limit: 4 * n_rays * ceil(n_samples / 32) + 4 * (n_rays / 1024 + 2), each part rounded up to
 *    256 bytes, must not exceed GNR_SAMPLE_STATIC_SCRATCH_BYTES (4 MiB of bit words plus one 4 KiB
 *    page for the block sums: 65536 rays x 512 samples fit, 65536 + 4096 rays x 512 do not);
 *    larger chunks are refused with an error, nothing is enqueued.
 *  - Preconditions are those of gnr_sample: with sampling_mode 1 the hull tables must have been
 *    uploaded for exactly ``n_samples`` (gnr_upload_hull_tables); otherwise the call is refused.
 *  - All five outputs are required device buffers owned by the caller: ``t_min[n]``, ``counts[n]``,
 *    ``offsets[n+1]``, ``ids[max_valid]`` and an 8-word ``status`` block (GNR_ST_* indices) that
 *    the call clears first and that reports an ``ids`` overflow.  Results equal gnr_sample's.
 *  - The first call on a device looks up the array's device address (with that device
 *    current); make that first call outside any stream capture.
 *  - All calls on one GPU share the array and it keeps the previous call's contents; the call
 *    rewrites every word it reads, so nothing stale leaks in, but two calls that overlap on
 *    the GPU (different streams, no dependency) race on it.  Serialise them. */
#define GNR_SAMPLE_STATIC_SCRATCH_BYTES ((4u << 20) + 4096u)
int gnr_sample_static(GnrModel* m, const float* rays, int64_t n_rays, int n_samples, int64_t max_valid,
                      float* t_min, int32_t* counts, int32_t* offsets, uint32_t* ids, int32_t* status,
                      void* stream);

/* Stage 2: density for the compacted samples of the last gnr_sample on this workspace:
 * ``sigma[i] = feature2density(compute_densityfeature(xyz_i))``; also the raw feature.
 * gridnerf_sequential.py:471-475,779-827,386-399. */
int gnr_density(GnrModel* m, const float* rays, int64_t n_rays, int n_samples, void* workspace,
                size_t workspace_bytes, int64_t max_valid, float* sigma_feature, float* sigma, void* stream);

/* Stage 3: raw2alpha + app_mask + second compaction (app/tools/utils.py:51-64,
 * gridnerf_sequential.py:477-479,493,501).  ``weights[i]`` per valid sample, ``acc[n]``,
 * ``depth[n]``, ``app_counts[n]``, ``app_offsets[n+1]`` (exclusive scan of app_counts),
 * ``app_index[j]`` = position in the valid list of appearance sample j.  The appearance list is
 * ordered inside groups of 32 consecutive rays: group g owns entries app_offsets[32 g] ..
 * app_offsets[min(32 g + 32, n)), first the first appearance sample of each of its rays (in ray
 * order), then the second ones, and so on; a ray's samples keep their order along the ray. */
int gnr_weights(GnrModel* m, const float* rays, int64_t n_rays, int n_samples, void* workspace,
                size_t workspace_bytes, int64_t max_valid, int64_t max_app, float* weights, float* acc,
                float* depth, int32_t* app_counts, int32_t* app_offsets, int32_t* app_index, void* stream);

/* Stages 2 + 3 in one pass (what gnr_render_chunk runs): density of the valid samples of the
 * last gnr_sample on this workspace, raw2alpha with the transmittance product in sample order,
 * early ray termination at GnrConfig.ert_transmittance (0 = none), and the appearance compaction.
 * Outputs as gnr_weights (samples after a ray's termination have weight 0); no sigma is kept.
 * With ``weights`` and ``app_index`` both null the pass writes only the samples above the appearance
 * threshold (what gnr_render_chunk does): the appearance list, counts, offsets, acc and depth are the same,
 * the workspace's per-sample weight array is then not filled. */
int gnr_march(GnrModel* m, const float* rays, int64_t n_rays, int n_samples, void* workspace,
              size_t workspace_bytes, int64_t max_valid, int64_t max_app, float* weights, float* acc,
              float* depth, int32_t* app_counts, int32_t* app_offsets, int32_t* app_index, void* stream);

/* Stage 4: compute_appfeature (gather + basis_mat) and MLPRender_Fea for the appearance
 * samples: ``app_features[j][app_dim]`` and ``rgb[j][3]``.  gridnerf_sequential.py:829-871,
 * app/models/mlp_render_fea.py:44-68. */
int gnr_appearance(GnrModel* m, const float* rays, int64_t n_rays, int n_samples, void* workspace,
                   size_t workspace_bytes, int64_t max_valid, int64_t max_app, float* app_features,
                   float* rgb, void* stream);

/* Stage 5: rgb_map = sum w * rgb (+ 1 - acc), clamp; depth_map.  gridnerf_sequential.py:493-501. */
int gnr_composite(GnrModel* m, int64_t n_rays, int white_bg, void* workspace, size_t workspace_bytes,
                  int64_t max_valid, int64_t max_app, int n_samples, float* rgb_map, float* depth_map,
                  void* stream);

/* ---- split-stage and point-mode entries ------------------------------------------------------
 * Building blocks for renderers that spread ONE field over several GPUs and exchange samples or
 * partial results with collectives: the reference's branch (block) parallel model
 * (app/models/gridnerf_parallel.py:279-338,765-859) and its tensor (channel) parallel model
 * (app/models/gridnerf_tensor_parallel.py:198-217,284-330).  The host composes them with
 * torch.distributed calls (landmark_b200/model_parallel.py). */

/* Normalised coordinates ``xyz[i][3]`` (normalize_coord, gridnerf_sequential.py:203-204) and ray
 * number of every valid sample of the last gnr_sample on this workspace. */
int gnr_valid_positions(GnrModel* m, const float* rays, int64_t n_rays, int n_samples, void* workspace,
                        size_t workspace_bytes, int64_t max_valid, float* xyz, int32_t* ray_index, void* stream);
/* Block routing: assign_blocks_to_samples (app/models/gridnerf_parallel.py:279-338; kernel version
 * dist_render/kernel/cuda_kernel/sampleray_gridsample/compute_assign_blocks_to_samples_norm_cuda_kernel.cu:19-74)
 * for a field cut into ``px x py`` blocks (block b = bx * py + by, at most 32), applied to the valid list
 * (``which_list`` 0, after gnr_sample) or the appearance list (1, after gnr_weights / gnr_weights_from_sigma
 * / gnr_march) of the workspace, fused with the grouping an all-to-all needs.  ``send_points`` receives the
 * block-local points grouped by block, block 0 first and list order inside a block (a stable partition):
 * rows of 3 floats (x, y local to the block, z) for the valid list, 6 floats (point, view direction) for the
 * appearance list; capacity = the list's capacity.  ``dest_row[i]`` = row of list entry i in that buffer (use
 * it to bring the owners' answers back into list order), ``counts[px*py]`` = rows per block (device int32),
 * ``block_of[i]`` (optional) = block of entry i.  Block indices and local coordinates have the bits of the
 * reference's torch arithmetic, except that x or y == 1 belongs to the last block instead of one past it.
 * Three launches on ``stream``, no host synchronisation; the first call on a model allocates 150 KB. */
int gnr_route_blocks(GnrModel* m, const float* rays, int64_t n_rays, int n_samples, void* workspace, size_t workspace_bytes,
                     int64_t max_valid, int64_t max_app, int which_list, int px, int py, float* send_points,
                     int32_t* dest_row, int32_t* counts, int32_t* block_of, void* stream);
/* compute_densityfeature + feature2density at explicit normalised points (block owner side of
 * gridnerf_parallel.py:765-790).  ``sigma_feature`` may be NULL. */
int gnr_density_points(GnrModel* m, const float* xyz, int64_t n, float* sigma_feature, float* sigma, void* stream);
/* raw2alpha + app_mask + compaction with sigma supplied by the caller (``sigma[max_valid]``, one
 * value per valid sample, as gathered from the block owners; gridnerf_parallel.py:791-800).
 * ``app_index[max_app]`` (optional) receives the appearance list. */
int gnr_weights_from_sigma(GnrModel* m, int64_t n_rays, int n_samples, void* workspace, size_t workspace_bytes,
                           int64_t max_valid, int64_t max_app, const float* sigma, int32_t* app_index, void* stream);
/* Block routing that ships ids instead of positions.  gnr_route_block_ids is gnr_route_blocks with one 32-bit id per row,
 * ``(ray_base + ray) << gnr_sample_bits(n_samples) | sample``, in place of the block-local point (and view direction):
 * a third (a sixth) of the bytes of a valid (appearance) sample on the wire.  The owner holds the rays and t_min of
 * every rank of the chunk in one table (rank r's first ray at its ray_base) and recomputes each position from its ray
 * with the SAMPLER's parametrisation and global box (``sampler``: the model the chunk was sampled with, on the same
 * device), then expresses it in the coordinates of its own block with the arithmetic of assign_blocks_to_samples
 * (app/models/gridnerf_parallel.py:296-327): gnr_density_list (sigma per id) and gnr_appearance_list (rgb per id; the
 * one-kernel appearance path in list mode, view direction = the ray's) give the bits of gnr_density_points /
 * gnr_appearance_rows on the rows gnr_route_blocks would have sent. */
int gnr_query_one_kernel_appearance(const GnrModel* m); /* 1 if gnr_render_chunk / gnr_appearance_list run the one-kernel path */
int gnr_route_block_ids(GnrModel* m, const float* rays, int64_t n_rays, int n_samples, void* workspace, size_t workspace_bytes,
                        int64_t max_valid, int64_t max_app, int which_list, int px, int py, uint32_t ray_base,
                        uint32_t* send_ids, int32_t* dest_row, int32_t* counts, void* stream);
int gnr_density_list(GnrModel* owner, const GnrModel* sampler, const float* rays_all, const float* t_min_all,
                     const uint32_t* ids, int64_t n, int n_samples, int px, int py, int block, float* sigma, void* stream);
int gnr_appearance_list(GnrModel* owner, const GnrModel* sampler, const float* rays_all, const float* t_min_all,
                        const uint32_t* ids, int64_t n, int n_samples, int px, int py, int block, void* scratch,
                        size_t scratch_bytes, float* rgb, void* stream);
/* gnr_weights_from_sigma for a caller whose sigma values still lie in the order they came back from the block owners:
 * the sigma of valid-list entry i is ``sigma_rows[rows[i]]`` (``rows`` = the dest_row output of gnr_route_blocks), read in
 * place.  Leaves the appearance list (ids, weights, counts, offsets) in the workspace for gnr_route_blocks /
 * gnr_composite_rgb; the per-sample weight array and the valid-list index of the entries are not produced. */
int gnr_weights_from_rows(GnrModel* m, int64_t n_rays, int n_samples, void* workspace, size_t workspace_bytes,
                          int64_t max_valid, int64_t max_app, const float* sigma_rows, const int32_t* rows, void* stream);
/* compute_appfeature only (gather + basis projection; on the tensor cores with mlp_mode 1/2, in fp32
 * on the CUDA cores with mode 0) for the appearance list of the workspace: with a channel slice of
 * the planes and the matching columns of basis_mat these are the partial sums a tensor-parallel
 * rank contributes (gridnerf_tensor_parallel.py:284-300).  ``features[n_features][app_dim]``
 * receives the first n_features rows of the list (the caller read the list length from the status
 * block; negative = max_app rows). */
int gnr_app_features(GnrModel* m, const float* rays, int64_t n_rays, int n_samples, void* workspace,
                     size_t workspace_bytes, int64_t max_valid, int64_t max_app, float* features, int64_t n_features,
                     void* stream);
/* Scratch for the two calls below (256-byte aligned, caller-allocated). */
int gnr_points_scratch_bytes(const GnrModel* m, int64_t n, size_t* bytes_h);
/* compute_appfeature + MLPRender_Fea at explicit points: ``xyz[n][3]`` normalised, ``view[n][3]``
 * -> ``rgb[n][3]`` (and optionally ``features[n][app_dim]``).  Block owner side of
 * gridnerf_parallel.py:801-859. */
int gnr_appearance_points(GnrModel* m, const float* xyz, const float* view, int64_t n, void* scratch,
                          size_t scratch_bytes, float* features, float* rgb, void* stream);
/* The same with the points as the rows gnr_route_blocks writes for an appearance list, ``rows[n][6]`` =
 * (x, y, z, view x, view y, view z): what a block owner receives from the all-to-all, read in place. */
int gnr_appearance_rows(GnrModel* m, const float* rows, int64_t n, void* scratch, size_t scratch_bytes, float* rgb,
                        void* stream);
/* compute_appfeature alone at explicit points: ``features[n][app_dim]`` = basis_mat(plane x line products) of
 * this model's appearance channels.  With a channel slice of the planes and the matching columns of basis_mat
 * these are the partial sums a tensor-parallel rank contributes for points that any rank sampled
 * (gridnerf_tensor_parallel.py:284-300).  Same scratch as gnr_appearance_points. */
int gnr_app_features_points(GnrModel* m, const float* xyz, int64_t n, void* scratch, size_t scratch_bytes,
                            float* features, void* stream);
/* Tensor-parallel exchange in fp16: ``features_h[n][32]`` (fp16, 64-byte rows, columns >= app_dim zero) = the partial
 * projection of this model's channel slice at ``xyz`` (rows of ``point_stride`` floats), on the tensor cores; needs
 * mlp_mode 2 and app_storage 1 with 16 / 32 / 48 padded channels per plane.  ``status``: 8 device words (zeroed here;
 * word GNR_ST_WAIT_EXPIRED is raised if a bounded wait of the kernel ran out).  No reference counterpart as a separate
 * entry: the reference sums fp32 products after an all-gather (gridnerf_tensor_parallel.py:284-300). */
int gnr_project_slice_points(GnrModel* m, const float* xyz, int point_stride, int64_t n, void* features_h, int32_t* status,
                             void* stream);
/* ``features[rows][app_dim]`` (fp32) = sum over ``n_parts`` buffers of fp16 rows of 32 (part w starts
 * ``w * part_stride_rows`` rows into ``parts_h``): the receiver's side of that exchange. */
int gnr_sum_partials(GnrModel* m, const void* parts_h, int n_parts, int64_t rows, int64_t part_stride_rows, float* features,
                     void* stream);
/* gnr_sum_partials + gnr_mlp_features in one kernel: rgb[n][3] of the points whose W partial rows lie in ``parts_h``
 * (summed in fp32, parts in order, inside the one-kernel appearance path) and whose view directions are columns 3..5
 * of ``rows6[n][6]`` (the rows gnr_route_blocks writes for an appearance list).  mlp_mode 2 only. */
int gnr_mlp_partial_rows(GnrModel* m, const void* parts_h, int n_parts, int64_t part_stride_rows, const float* rows6,
                         int64_t n, void* scratch, size_t scratch_bytes, float* rgb, void* stream);
/* MLPRender_Fea alone on explicit ``features[n][app_dim]`` and ``view[n][3]`` (the sample slice a
 * tensor-parallel rank owns after the reduction, gridnerf_tensor_parallel.py:301-325). */
int gnr_mlp_features(GnrModel* m, const float* features, const float* view, int64_t n, void* scratch,
                     size_t scratch_bytes, float* rgb, void* stream);
/* Compositing with per-appearance-sample colours supplied by the caller
 * (``rgb_samples[n_rgb][3]`` in the order of the workspace's appearance list). */
int gnr_composite_rgb(GnrModel* m, int64_t n_rays, int white_bg, void* workspace, size_t workspace_bytes,
                      int64_t max_valid, int64_t max_app, int n_samples, const float* rgb_samples, int64_t n_rgb,
                      float* rgb_map, float* depth_map, void* stream);

/* Per-stage timing with CUDA events recorded on the launching stream around every stage of
 * gnr_render_chunk / gnr_render_host (the counterpart of the reference's PipeStagesProfiler,
 * dist_render/comm/profiler.py:18-69, at kernel granularity).  gnr_profile_collect waits for
 * the recorded events, adds the elapsed milliseconds per stage into ``stage_ms_h[GNR_STAGE_COUNT]``
 * and the number of kernel launches per stage into ``launches_h[GNR_STAGE_COUNT]``, then clears. */
enum {
  GNR_STAGE_SAMPLE = 0,     /* sampling + occupancy test (mask words, counts)             */
  GNR_STAGE_COMPACT = 1,    /* scan + compaction of the valid samples                     */
  GNR_STAGE_DENSITY = 2,    /* density feature gather                                     */
  GNR_STAGE_WEIGHTS = 3,    /* transmittance / weights                                    */
  GNR_STAGE_COMPACT_APP = 4,/* scan + compaction of the appearance samples                */
  GNR_STAGE_APP_GATHER = 5, /* appearance gather + basis projection                       */
  GNR_STAGE_MLP = 6,        /* appearance MLP                                             */
  GNR_STAGE_COMPOSITE = 7,  /* final compositing                                          */
  GNR_STAGE_COUNT = 8
};
int gnr_profile_enable(GnrModel* m, int on);
int gnr_profile_collect(GnrModel* m, float* stage_ms_h, int64_t* launches_h);

/* Measurement helper for roofline figures: the rate (GB/s, whole GPU) at which the L1 caches deliver
 * 256-bit loads that hit in L1 into registers, measured with a small kernel that re-reads a per-CTA
 * buffer ``iters`` times (CUDA events around one launch).  The feature gathers of this library are bound
 * by that path, not by HBM, so their roofline fractions are quoted against this number.  Host call;
 * allocates and frees its own few megabytes; synchronises the device. */
int gnr_measure_l1_bandwidth(int device, int iters, float* gb_per_s_h);

/* Test hook for the bounded device-side waits of the tensor-core kernels.  ``wait_limit`` > 0 replaces
 * the number of polls a wait may take (default 2^20); with ``expire`` != 0 one group of one CTA of every
 * following tensor-core launch leaves out the step its next wait depends on (the bulk copy of its first
 * tile in the MLP kernel, the commit of its first projection in the fused kernel), so that this wait
 * runs out: the group raises status[GNR_ST_WAIT_EXPIRED] and stops, the kernel frees its tensor memory
 * and returns, and the context stays usable.  ``expire`` = 0, ``wait_limit`` = 0 restores normal
 * operation.  Nothing in this hook faults, traps or spins without bound. */
int gnr_debug_wait(GnrModel* m, int expire, int wait_limit);

/* Measurement aid for the fused appearance kernel: with ``on`` != 0 the following launches let one thread
 * per group of the middle CTA sum the clock cycles it spends in each phase of a tile (store A0, projection,
 * gather behind it, wait, encoding, layer 1, ...); ``on`` == 0 synchronises, copies the last launch's sums
 * to ``cycles_h[64]`` ([group][16 phases], unused entries zero) and switches the timer off. */
int gnr_debug_phase_cycles(GnrModel* m, int on, long long* cycles_h);

/* Copy the 8-word status block of a workspace to the host (synchronises the stream). */
int gnr_read_status(const void* workspace, int32_t* status_h, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GRIDNERF_B200_H */
