// C-ABI entry points: model lifetime, parameter upload / layout conversion, workspace layout,
// the per-chunk forward and its stage-wise pieces.
#include <cuda_fp16.h>
#include <stdarg.h>
#include <string.h>

#include <new>
#include <vector>

#include "gnr_internal.cuh"

// ---------------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------------
static thread_local char g_error[512] = "";

void gnr_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

extern "C" const char* gnr_last_error(void) { return g_error; }
extern "C" int gnr_version(void) { return 100; }

// Event-pair profiler: one span per stage per chunk, summed at collect time.
struct GnrProfiler {
  struct Span {
    int stage;
    int launches;
    cudaEvent_t a, b;
  };
  std::vector<Span> spans;
  std::vector<cudaEvent_t> pool;
  cudaEvent_t get() {
    if (!pool.empty()) {
      cudaEvent_t e = pool.back();
      pool.pop_back();
      return e;
    }
    cudaEvent_t e;
    cudaEventCreate(&e);
    return e;
  }
  void begin(int stage, int launches, cudaStream_t st) {
    Span s{stage, launches, get(), get()};
    cudaEventRecord(s.a, st);
    spans.push_back(s);
  }
  void end(cudaStream_t st) { cudaEventRecord(spans.back().b, st); }
  ~GnrProfiler() {
    for (auto& s : spans) {
      cudaEventDestroy(s.a);
      cudaEventDestroy(s.b);
    }
    for (auto e : pool) cudaEventDestroy(e);
  }
};

#define GNR_LAUNCH_OK(call)                                                                  \
  do {                                                                                       \
    int _e = (call);                                                                         \
    if (_e > 0) {                                                                            \
      gnr_set_error("%s: %s", #call, cudaGetErrorString((cudaError_t)_e));                   \
      return -2;                                                                             \
    }                                                                                        \
    if (_e < 0) return _e;                                                                   \
  } while (0)

namespace {

struct StageScope {
  GnrProfiler* p;
  cudaStream_t st;
  StageScope(GnrModel* m, int stage, int launches, cudaStream_t s) : p(m->prof), st(s) {
    if (p) p->begin(stage, launches, st);
  }
  ~StageScope() {
    if (p) p->end(st);
  }
};

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct DeviceGuard {
  int prev;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
  }
  ~DeviceGuard() { cudaSetDevice(prev); }
};

// ---- layout conversion kernels -------------------------------------------------------------
// [C][P] (P = H*W or L) -> [P][Cp], zero padded channels.  A 32x32 tile goes through shared
// memory so that both the read and the write are coalesced.
__global__ void to_channel_last_kernel(const float* __restrict__ src, float* __restrict__ dst, int C, int Cp, long long P) {
  __shared__ float tile[32][33];
  const long long p0 = (long long)blockIdx.x * 32;
  const int c0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int c = c0 + r;
    const long long p = p0 + threadIdx.x;
    tile[r][threadIdx.x] = (c < C && p < P) ? src[(long long)c * P + p] : 0.0f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const long long p = p0 + r;
    const int c = c0 + threadIdx.x;
    if (p < P && c < Cp) dst[p * Cp + c] = tile[threadIdx.x][r];
  }
}

// Same, to fp16 (appearance planes with GnrConfig.app_storage == 1).
__global__ void to_channel_last_half_kernel(const float* __restrict__ src, __half* __restrict__ dst, int C, int Cp, long long P) {
  __shared__ float tile[32][33];
  const long long p0 = (long long)blockIdx.x * 32;
  const int c0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int c = c0 + r;
    const long long p = p0 + threadIdx.x;
    tile[r][threadIdx.x] = (c < C && p < P) ? src[(long long)c * P + p] : 0.0f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const long long p = p0 + r;
    const int c = c0 + threadIdx.x;
    if (p < P && c < Cp) dst[p * Cp + c] = __float2half_rn(tile[threadIdx.x][r]);
  }
}

__global__ void pack_bits_kernel(const uint8_t* __restrict__ vol, uint32_t* __restrict__ bits, long long n_vox, long long n_words) {
  long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= n_words) return;
  uint32_t v = 0;
  for (int b = 0; b < 32; ++b) {
    long long i = w * 32 + b;
    if (i < n_vox && vol[i]) v |= (1u << b);
  }
  bits[w] = v;
}

__global__ void transpose_pad_kernel(const float* __restrict__ w, float* __restrict__ wt, int out_f, int in_f, int in_pad) {
  // w [out_f][in_f] -> wt [in_pad][out_f]
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= in_pad * out_f) return;
  int k = i / out_f, n = i - k * out_f;
  wt[i] = (k < in_f) ? w[n * in_f + k] : 0.0f;
}

__global__ void copy_or_zero_kernel(const float* __restrict__ src, float* __restrict__ dst, int n_src, int n_dst) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_dst) dst[i] = (src && i < n_src) ? src[i] : 0.0f;
}

// basis_mat.weight [app_dim][n_pairs * C] -> blocked [pair][c4][t = 4 j + e][28] (+8 pad per block)
__global__ void block_basis_kernel(const float* __restrict__ w, float* __restrict__ dst, int app_dim, int n_pairs, int C, int J) {
  const int blk = 4 * J * 28 + 8;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs * 4 * blk) return;
  int pc = i / blk, r = i - pc * blk;
  int pair = pc >> 2, c4 = pc & 3;
  float v = 0.0f;
  if (r < 4 * J * 28) {
    int t = r / 28, o = r - t * 28;
    int j = t >> 2, e = t & 3;
    int c = 16 * j + 4 * c4 + e;
    if (o < app_dim && c < C) v = w[(long long)o * (n_pairs * C) + pair * C + c];
  }
  dst[i] = v;
}

int free_dev(void* p) {
  if (p) cudaFree(p);
  return 0;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// lifetime
// ---------------------------------------------------------------------------------------------
extern "C" int gnr_create(const GnrConfig* cfg, int device, GnrModel** out) {
  if (!cfg || !out) {
    gnr_set_error("gnr_create: null argument");
    return -1;
  }
  if (cfg->n_pairs < 1 || cfg->n_pairs > GNR_MAX_PLANES) {
    gnr_set_error("gnr_create: n_pairs %d outside [1, %d]", cfg->n_pairs, GNR_MAX_PLANES);
    return -1;
  }
  if (cfg->app_dim < 1 || cfg->app_dim > 28) {
    gnr_set_error("gnr_create: app_dim %d outside [1, 28]", cfg->app_dim);
    return -1;
  }
  if (cfg->n_density < 1 || cfg->n_density > 64 || cfg->n_app < 1 || cfg->n_app > 64) {
    gnr_set_error("gnr_create: channels per plane must be in [1, 64] (density %d, appearance %d)", cfg->n_density, cfg->n_app);
    return -1;
  }
  if (cfg->sampling_mode != 0 && cfg->sampling_mode != 1) {
    gnr_set_error("gnr_create: sampling_mode %d (0 = dense, 1 = hull)", cfg->sampling_mode);
    return -1;
  }
  if (cfg->app_storage != 0 &&
      (cfg->app_storage != 1 || cfg->mlp_mode != 2 || cfg->n_app > 48 || cfg->app_dim > 27)) {
    // (33..48 channels: every appearance path; fewer, a channel slice: gnr_project_slice_points only)
    gnr_set_error("gnr_create: app_storage %d: fp16 appearance planes need mlp_mode 2 (got %d) and at most 48 appearance channels (got %d)",
                  cfg->app_storage, cfg->mlp_mode, cfg->n_app);
    return -1;
  }
  if (cfg->den_storage != 0 && (cfg->den_storage != 1 || cfg->n_density > 16)) {
    gnr_set_error("gnr_create: den_storage %d: fp16 density planes are implemented for up to 16 channels (got %d)",
                  cfg->den_storage, cfg->n_density);
    return -1;
  }
  if (cfg->fea_pe < 0 || cfg->fea_pe > 8 || cfg->view_pe < 0 || cfg->view_pe > 8) {
    gnr_set_error("gnr_create: fea_pe %d / view_pe %d outside [0, 8]", cfg->fea_pe, cfg->view_pe);
    return -1;
  }
  int n_dev = 0;
  GNR_CUDA_OK(cudaGetDeviceCount(&n_dev));
  if (device < 0 || device >= n_dev) {
    gnr_set_error("gnr_create: device %d not present (%d devices)", device, n_dev);
    return -1;
  }
  cudaDeviceProp prop;
  GNR_CUDA_OK(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    gnr_set_error("gnr_create: device %d is sm_%d%d; this library contains sm_100a code only", device, prop.major, prop.minor);
    return -1;
  }
  GnrModel* m = new (std::nothrow) GnrModel();
  if (!m) {
    gnr_set_error("gnr_create: out of host memory");
    return -1;
  }
  memset(m, 0, sizeof(*m));
  m->cfg = *cfg;
  m->device = device;
  m->sm_count = prop.multiProcessorCount > 0 ? prop.multiProcessorCount : GNR_SM_COUNT_FALLBACK;
  const int A = cfg->app_dim, V = cfg->view_pe > 0 ? cfg->view_pe : 0;
  m->mlp.in_dim = A + 3 + 2 * cfg->fea_pe * A + 2 * V * 3;
  m->mlp.k1_pad = (m->mlp.in_dim + 7) / 8 * 8;
  m->mlp.n_prod = cfg->n_pairs * ((cfg->n_app + 15) / 16 * 16);
  *out = m;
  return 0;
}

extern "C" int gnr_destroy(GnrModel* m) {
  if (!m) return 0;
  DeviceGuard g(m->device);
  cudaDeviceSynchronize();
  for (int i = 0; i < GNR_MAX_PLANES; ++i) {
    free_dev(m->den_plane_buf[i]);
    free_dev(m->den_line_buf[i]);
    free_dev(m->app_plane_buf[i]);
    free_dev(m->app_line_buf[i]);
  }
  free_dev(m->den_lattice);
  free_dev(m->app_lattice);
  free_dev(m->mlp.basis_raw);
  free_dev(m->debug_prof);
  free_dev(m->route_scratch);
  free_dev(m->alpha_bits);
  free_dev(m->alpha_coarse);
  free_dev(m->alpha_full);
  free_dev(m->hull_near_term);
  free_dev(m->hull_u);
  free_dev(m->mlp.basis_blocked);
  free_dev(m->mlp.w1t);
  free_dev(m->mlp.w2t);
  free_dev(m->mlp.w3);
  free_dev(m->mlp.b1);
  free_dev(m->mlp.b2);
  free_dev(m->mlp.b3);
  free_dev(m->mlp.tc_image);
  free_dev(m->host_ws);
  free_dev(m->host_rays);
  free_dev(m->host_rgb);
  free_dev(m->host_depth);
  if (m->host_status) cudaFreeHost(m->host_status);
  delete m->prof;
  for (int i = 0; i < 2; ++i) {
    if (m->host_streams[i]) cudaStreamDestroy(m->host_streams[i]);
    if (m->host_events[i]) cudaEventDestroy(m->host_events[i]);
  }
  delete m;
  return 0;
}

// ---------------------------------------------------------------------------------------------
// uploads
// ---------------------------------------------------------------------------------------------
static int padded_channels(int C) { return (C + 15) / 16 * 16; }

extern "C" int gnr_upload_plane(GnrModel* m, int kind, int idx, const float* src, int C, int H, int W, int axis_x,
                                int axis_y, void* stream) {
  if (!m || !src || kind < 0 || kind > 1 || idx < 0 || idx >= m->cfg.n_pairs || H < 1 || W < 1 ||
      axis_x < 0 || axis_x > 2 || axis_y < 0 || axis_y > 2) {
    gnr_set_error("gnr_upload_plane: bad argument (kind %d idx %d C %d H %d W %d)", kind, idx, C, H, W);
    return -1;
  }
  if (H < 2 || W < 2 || (long long)H * W * ((C + 15) / 16 * 4) > 0x7fffffffLL) {
    gnr_set_error("gnr_upload_plane: plane %dx%d must be at least 2x2 and fit 32-bit texel offsets", W, H);
    return -1;
  }
  const int expect = kind == 0 ? m->cfg.n_density : m->cfg.n_app;
  if (C != expect) {
    gnr_set_error("gnr_upload_plane: plane %d of kind %d has %d channels, config says %d", idx, kind, C, expect);
    return -1;
  }
  DeviceGuard g(m->device);
  const int Cp = padded_channels(C);
  float** buf = kind == 0 ? &m->den_plane_buf[idx] : &m->app_plane_buf[idx];
  GnrPlane* pl = kind == 0 ? &m->den[idx] : &m->app[idx];
  const long long P = (long long)H * W;
  const bool half = (kind == 1 && m->cfg.app_storage == 1) || (kind == 0 && m->cfg.den_storage == 1);
  const size_t need = (size_t)P * Cp * (half ? sizeof(__half) : sizeof(float));
  if (*buf == nullptr || m->plane_bytes[kind][idx] != need) {
    free_dev(*buf);
    *buf = nullptr;
    m->plane_bytes[kind][idx] = 0;
    GNR_CUDA_OK(cudaMalloc(buf, need));
    m->plane_bytes[kind][idx] = need;
  }
  dim3 grid((unsigned)((P + 31) / 32), (unsigned)((Cp + 31) / 32)), block(32, 8);
  if (half)
    to_channel_last_half_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(src, reinterpret_cast<__half*>(*buf), C, Cp, P);
  else
    to_channel_last_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(src, *buf, C, Cp, P);
  GNR_CUDA_OK(cudaGetLastError());
  if (kind == 0) m->lat_valid = 0;  // a lattice built from the previous planes no longer describes the field
  if (kind == 1) m->app_lat_valid = 0;
  pl->plane = *buf;
  pl->H = H;
  pl->W = W;
  pl->fw = (float)(W - 1);
  pl->fh = (float)(H - 1);
  pl->C = Cp;
  pl->mat0 = axis_x;
  pl->mat1 = axis_y;
  return 0;
}

extern "C" int gnr_upload_line(GnrModel* m, int kind, int idx, const float* src, int C, int Ln, int axis, void* stream) {
  if (!m || !src || kind < 0 || kind > 1 || idx < 0 || idx >= m->cfg.n_pairs || Ln < 1 || axis < 0 || axis > 2) {
    gnr_set_error("gnr_upload_line: bad argument (kind %d idx %d C %d L %d)", kind, idx, C, Ln);
    return -1;
  }
  if (Ln < 2) {
    gnr_set_error("gnr_upload_line: a line needs at least 2 entries");
    return -1;
  }
  const int expect = kind == 0 ? m->cfg.n_density : m->cfg.n_app;
  if (C != expect) {
    gnr_set_error("gnr_upload_line: line %d of kind %d has %d channels, config says %d", idx, kind, C, expect);
    return -1;
  }
  DeviceGuard g(m->device);
  const int Cp = padded_channels(C);
  float** buf = kind == 0 ? &m->den_line_buf[idx] : &m->app_line_buf[idx];
  GnrPlane* pl = kind == 0 ? &m->den[idx] : &m->app[idx];
  const bool half = (kind == 1 && m->cfg.app_storage == 1) || (kind == 0 && m->cfg.den_storage == 1);
  const size_t need = (size_t)Ln * Cp * (half ? sizeof(__half) : sizeof(float));
  if (*buf == nullptr || m->line_bytes[kind][idx] != need) {
    free_dev(*buf);
    *buf = nullptr;
    m->line_bytes[kind][idx] = 0;
    GNR_CUDA_OK(cudaMalloc(buf, need));
    m->line_bytes[kind][idx] = need;
  }
  dim3 grid((unsigned)((Ln + 31) / 32), (unsigned)((Cp + 31) / 32)), block(32, 8);
  if (half)
    to_channel_last_half_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(src, reinterpret_cast<__half*>(*buf), C, Cp,
                                                                          (long long)Ln);
  else
    to_channel_last_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(src, *buf, C, Cp, (long long)Ln);
  GNR_CUDA_OK(cudaGetLastError());
  if (kind == 0) m->lat_valid = 0;
  if (kind == 1) m->app_lat_valid = 0;
  pl->line = *buf;
  pl->L = Ln;
  pl->fl = (float)(Ln - 1);
  pl->vec = axis;
  return 0;
}

// Coarse occupancy: block (bx, by, bz) covers mask cells [4 b, 4 b + 4] on each axis (its own 4 and
// the first cell of the next block: a trilinear test whose lower corner lies in the block reads
// those).  A clear bit therefore proves that the fine test of any such sample sums to zero.
__global__ void coarse_bits_kernel(const uint32_t* __restrict__ bits, int D, int H, int W, int cD, int cH, int cW,
                                   uint32_t* __restrict__ coarse) {
  const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool in_range = c < (long long)cD * cH * cW;
  bool any = false;
  if (in_range) {
    const int bx = (int)(c % cW), by = (int)((c / cW) % cH), bz = (int)(c / ((long long)cW * cH));
    for (int z = 4 * bz; z <= 4 * bz + 4 && z < D && !any; ++z)
      for (int y = 4 * by; y <= 4 * by + 4 && y < H && !any; ++y)
        for (int x = 4 * bx; x <= 4 * bx + 4 && x < W; ++x) {
          const uint32_t bit = (uint32_t)(((long long)z * H + y) * W + x);
          if ((bits[bit >> 5] >> (bit & 31)) & 1u) {
            any = true;
            break;
          }
        }
  }
  const uint32_t word = __ballot_sync(0xffffffffu, any);  // 32 consecutive blocks = one word
  if ((threadIdx.x & 31) == 0 && c < (((long long)cD * cH * cW + 31) / 32) * 32) coarse[c >> 5] = word;
}

// The opposite bound: block (bx, by, bz) is "full" if every mask cell of [4 b, 4 b + 4]^3 exists and
// is set.  A sample whose lower corner lies in a full block then has that corner occupied.
__global__ void full_bits_kernel(const uint32_t* __restrict__ bits, int D, int H, int W, int cD, int cH, int cW,
                                 uint32_t* __restrict__ full) {
  const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  bool all = c < (long long)cD * cH * cW;
  if (all) {
    const int bx = (int)(c % cW), by = (int)((c / cW) % cH), bz = (int)(c / ((long long)cW * cH));
    all = 4 * bx + 4 < W && 4 * by + 4 < H && 4 * bz + 4 < D;
    for (int z = 4 * bz; all && z <= 4 * bz + 4; ++z)
      for (int y = 4 * by; all && y <= 4 * by + 4; ++y)
        for (int x = 4 * bx; x <= 4 * bx + 4; ++x) {
          const uint32_t bit = (uint32_t)(((long long)z * H + y) * W + x);
          if (!((bits[bit >> 5] >> (bit & 31)) & 1u)) {
            all = false;
            break;
          }
        }
  }
  const uint32_t word = __ballot_sync(0xffffffffu, all);
  if ((threadIdx.x & 31) == 0 && c < (((long long)cD * cH * cW + 31) / 32) * 32) full[c >> 5] = word;
}

extern "C" int gnr_upload_alpha_mask(GnrModel* m, const uint8_t* vol, int D, int H, int W, const float* aabb_h,
                                     const float* inv_size_h, void* stream) {
  if (!m) {
    gnr_set_error("gnr_upload_alpha_mask: null model");
    return -1;
  }
  DeviceGuard g(m->device);
  free_dev(m->alpha_bits);
  free_dev(m->alpha_coarse);
  free_dev(m->alpha_full);
  m->alpha_bits = m->alpha_coarse = m->alpha_full = nullptr;
  m->aD = m->aH = m->aW = 0;
  if (!vol) return 0;
  if (D < 1 || H < 1 || W < 1 || !aabb_h || !inv_size_h || (long long)D * H * W > 0xffffffffLL) {
    gnr_set_error("gnr_upload_alpha_mask: bad volume %dx%dx%d", D, H, W);
    return -1;
  }
  const long long n_vox = (long long)D * H * W, n_words = (n_vox + 31) / 32;
  GNR_CUDA_OK(cudaMalloc(&m->alpha_bits, (size_t)n_words * sizeof(uint32_t)));
  pack_bits_kernel<<<(unsigned)((n_words + 255) / 256), 256, 0, (cudaStream_t)stream>>>(vol, m->alpha_bits, n_vox, n_words);
  GNR_CUDA_OK(cudaGetLastError());
  {
    const int cD = (D + 3) / 4, cH = (H + 3) / 4, cW = (W + 3) / 4;
    const long long n_blocks = (long long)cD * cH * cW, n_cwords = (n_blocks + 31) / 32;
    GNR_CUDA_OK(cudaMalloc(&m->alpha_coarse, (size_t)n_cwords * sizeof(uint32_t)));
    coarse_bits_kernel<<<(unsigned)((n_cwords * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(m->alpha_bits, D, H, W, cD, cH,
                                                                                            cW, m->alpha_coarse);
    GNR_CUDA_OK(cudaGetLastError());
    GNR_CUDA_OK(cudaMalloc(&m->alpha_full, (size_t)n_cwords * sizeof(uint32_t)));
    full_bits_kernel<<<(unsigned)((n_cwords * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(m->alpha_bits, D, H, W, cD, cH, cW,
                                                                                          m->alpha_full);
    GNR_CUDA_OK(cudaGetLastError());
  }
  m->aD = D;
  m->aH = H;
  m->aW = W;
  for (int a = 0; a < 3; ++a) {
    m->a_lo[a] = aabb_h[a];
    m->a_inv[a] = inv_size_h[a];
  }
  return 0;
}

extern "C" int gnr_upload_hull_tables(GnrModel* m, int n_samples, const float* near_term, const float* u, void* stream) {
  if (!m || n_samples < 1 || !near_term || !u) {
    gnr_set_error("gnr_upload_hull_tables: bad argument");
    return -1;
  }
  DeviceGuard g(m->device);
  free_dev(m->hull_near_term);
  free_dev(m->hull_u);
  m->hull_near_term = m->hull_u = nullptr;
  m->hull_samples = 0;
  GNR_CUDA_OK(cudaMalloc(&m->hull_near_term, (size_t)n_samples * 4));
  GNR_CUDA_OK(cudaMalloc(&m->hull_u, (size_t)n_samples * 4));
  GNR_CUDA_OK(cudaMemcpyAsync(m->hull_near_term, near_term, (size_t)n_samples * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  GNR_CUDA_OK(cudaMemcpyAsync(m->hull_u, u, (size_t)n_samples * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  m->hull_samples = n_samples;
  return 0;
}

extern "C" int gnr_upload_mlp(GnrModel* m, const float* basis_w, const float* w1, const float* b1, const float* w2,
                              const float* b2, const float* w3, const float* b3, void* stream) {
  if (!m || !basis_w || !w1 || !w2 || !w3) {
    gnr_set_error("gnr_upload_mlp: null weight pointer");
    return -1;
  }
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  GnrMlp& q = m->mlp;
  const int Hd = m->cfg.hidden, J = padded_channels(m->cfg.n_app) / 16;
  const int n_basis = m->cfg.n_pairs * 4 * (4 * J * 28 + 8);
  free_dev(q.basis_raw);
  q.basis_raw = nullptr;
  m->app_lat_valid = 0;  // the lattice bakes the basis matrix in
  free_dev(q.basis_blocked);
  free_dev(q.w1t);
  free_dev(q.w2t);
  free_dev(q.w3);
  free_dev(q.b1);
  free_dev(q.b2);
  free_dev(q.b3);
  q.basis_blocked = q.w1t = q.w2t = q.w3 = q.b1 = q.b2 = q.b3 = nullptr;
  {
    const size_t raw = (size_t)m->cfg.app_dim * m->cfg.n_pairs * m->cfg.n_app * sizeof(float);
    GNR_CUDA_OK(cudaMalloc(&q.basis_raw, raw));
    GNR_CUDA_OK(cudaMemcpyAsync(q.basis_raw, basis_w, raw, cudaMemcpyDeviceToDevice, st));
  }
  GNR_CUDA_OK(cudaMalloc(&q.basis_blocked, (size_t)n_basis * sizeof(float)));
  GNR_CUDA_OK(cudaMalloc(&q.w1t, (size_t)q.k1_pad * Hd * sizeof(float)));
  GNR_CUDA_OK(cudaMalloc(&q.w2t, (size_t)Hd * Hd * sizeof(float)));
  GNR_CUDA_OK(cudaMalloc(&q.w3, (size_t)3 * Hd * sizeof(float)));
  GNR_CUDA_OK(cudaMalloc(&q.b1, (size_t)Hd * sizeof(float)));
  GNR_CUDA_OK(cudaMalloc(&q.b2, (size_t)Hd * sizeof(float)));
  GNR_CUDA_OK(cudaMalloc(&q.b3, 4 * sizeof(float)));
  block_basis_kernel<<<(n_basis + 255) / 256, 256, 0, st>>>(basis_w, q.basis_blocked, m->cfg.app_dim, m->cfg.n_pairs,
                                                           m->cfg.n_app, J);
  transpose_pad_kernel<<<(q.k1_pad * Hd + 255) / 256, 256, 0, st>>>(w1, q.w1t, Hd, q.in_dim, q.k1_pad);
  transpose_pad_kernel<<<(Hd * Hd + 255) / 256, 256, 0, st>>>(w2, q.w2t, Hd, Hd, Hd);
  copy_or_zero_kernel<<<(3 * Hd + 255) / 256, 256, 0, st>>>(w3, q.w3, 3 * Hd, 3 * Hd);
  copy_or_zero_kernel<<<(Hd + 255) / 256, 256, 0, st>>>(b1, q.b1, Hd, Hd);
  copy_or_zero_kernel<<<(Hd + 255) / 256, 256, 0, st>>>(b2, q.b2, Hd, Hd);
  copy_or_zero_kernel<<<1, 32, 0, st>>>(b3, q.b3, 3, 4);
  GNR_CUDA_OK(cudaGetLastError());
  if (m->cfg.mlp_mode != 0) return gnr_mlp_tc_prepare(m, basis_w, w1, w2, w3, st);
  return 0;
}

extern "C" int gnr_build_density_lattice(GnrModel* m, int enable, void* stream) {
  if (!m) {
    gnr_set_error("gnr_build_density_lattice: null model");
    return -1;
  }
  DeviceGuard g(m->device);
  if (!enable) {
    if (m->den_lattice) {
      cudaDeviceSynchronize();  // kernels in flight may still read it
      free_dev(m->den_lattice);
    }
    m->den_lattice = nullptr;
    m->den_lattice_bytes = 0;
    m->lat_valid = 0;
    return 0;
  }
  int dims[3];
  if (gnr_lattice_dims(m, dims)) return -1;
  const size_t need = (size_t)dims[0] * dims[1] * dims[2] * sizeof(float);
  if (!m->den_lattice || m->den_lattice_bytes != need) {
    if (m->den_lattice) cudaDeviceSynchronize();
    free_dev(m->den_lattice);
    m->den_lattice = nullptr;
    m->den_lattice_bytes = 0;
    GNR_CUDA_OK(cudaMalloc(&m->den_lattice, need));
    m->den_lattice_bytes = need;
  }
  for (int a = 0; a < 3; ++a) m->lat_dims[a] = dims[a];
  GNR_LAUNCH_OK(launch_build_lattice(m, m->den_lattice, (cudaStream_t)stream));
  m->lat_valid = 1;
  return 0;
}

extern "C" int gnr_build_appearance_lattice(GnrModel* m, int enable, void* stream) {
  if (!m) {
    gnr_set_error("gnr_build_appearance_lattice: null model");
    return -1;
  }
  DeviceGuard g(m->device);
  if (!enable) {
    if (m->app_lattice) {
      cudaDeviceSynchronize();  // kernels in flight may still read it
      free_dev(m->app_lattice);
    }
    m->app_lattice = nullptr;
    m->app_lattice_bytes = 0;
    m->app_lat_valid = 0;
    return 0;
  }
  if (m->cfg.mlp_mode != 2 || m->cfg.n_pairs != 3) {
    gnr_set_error("gnr_build_appearance_lattice: needs mlp_mode 2 and three plane/line pairs (got mode %d, %d pairs)",
                  m->cfg.mlp_mode, m->cfg.n_pairs);
    return -1;
  }
  int dims[3];
  if (gnr_app_lattice_dims(m, dims)) return -1;
  const size_t need = (size_t)dims[0] * dims[1] * dims[2] * 32 * sizeof(__half);
  if (!m->app_lattice || m->app_lattice_bytes != need) {
    if (m->app_lattice) cudaDeviceSynchronize();
    free_dev(m->app_lattice);
    m->app_lattice = nullptr;
    m->app_lattice_bytes = 0;
    size_t free_b = 0, total_b = 0;
    GNR_CUDA_OK(cudaMemGetInfo(&free_b, &total_b));
    if (need + ((size_t)1 << 30) > free_b) {
      gnr_set_error("gnr_build_appearance_lattice: the lattice of %dx%dx%d points needs %.1f GB, %.1f GB are free",
                    dims[0], dims[1], dims[2], need / 1e9, free_b / 1e9);
      return -1;
    }
    GNR_CUDA_OK(cudaMalloc(&m->app_lattice, need));
    m->app_lattice_bytes = need;
  }
  for (int a = 0; a < 3; ++a) m->app_lat_dims[a] = dims[a];
  GNR_LAUNCH_OK(launch_build_app_lattice(m, m->app_lattice, (cudaStream_t)stream));
  m->app_lat_valid = 1;
  return 0;
}

// ---------------------------------------------------------------------------------------------
// workspace
// ---------------------------------------------------------------------------------------------
extern "C" int gnr_sample_bits(int n_samples) {
  int b = 1;
  while ((1 << b) < n_samples) ++b;
  return b;
}

GnrWs gnr_ws_layout(const GnrModel* m, int64_t n, int S, int64_t max_valid, int64_t max_app) {
  GnrWs L;
  memset(&L, 0, sizeof(L));
  const size_t words = (size_t)(S + 31) / 32;
  const size_t n_blocks = (size_t)(n + 1023) / 1024 + 1;
  L.feat_stride = (m->cfg.app_dim + 3) / 4 * 4;
  L.max_valid = max_valid;
  L.max_app = max_app;
  L.n_rays = n;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t at = off;
    off = align_up(off + bytes, 256);
    return at;
  };
  L.status = take(GNR_ST_WORDS * sizeof(int32_t));
  L.t_min = take((size_t)n * 4);
  L.words = take((size_t)n * words * 4);
  L.counts = take((size_t)n * 4);
  L.offsets = take((size_t)(n + 1) * 4);
  L.block_sums = take(n_blocks * 4);
  L.ids = take((size_t)max_valid * 4);
  L.sigma_feat = take((size_t)max_valid * 4);
  L.sigma = take((size_t)max_valid * 4);
  L.weight = take((size_t)max_valid * 4);
  L.acc = take((size_t)n * 4);
  L.depth = take((size_t)n * 4);
  L.app_counts = take((size_t)n * 4);
  L.app_offsets = take((size_t)(n + 1) * 4);
  L.app_index = take((size_t)max_app * 4);
  L.app_ids = take((size_t)max_app * 4);     // ray << kbits | sample of every appearance entry
  L.app_weight = take((size_t)max_app * 4);  // its compositing weight
  L.app_feat = take((size_t)max_app * L.feat_stride * 4);
  L.app_rgb = take((size_t)max_app * 3 * 4);
  if (gnr_tc_basis_fused(m)) {
    const int terms = m->cfg.mlp_mode == 1 ? 2 : 1;
    const size_t tiles = (size_t)(max_app + 127) / 128;
    L.app_prod_tile = gnr_tc_tile_bytes(m);
    L.app_prod_image = align_up(tiles * (size_t)L.app_prod_tile, 256);
    L.app_prod = take(L.app_prod_image * terms);
  }
  L.total = off;
  return L;
}

GnrSampleParams gnr_sample_params(const GnrModel* m, int S) {
  GnrSampleParams p;
  memset(&p, 0, sizeof(p));
  for (int a = 0; a < 3; ++a) {
    p.lo[a] = m->cfg.aabb[a];
    p.hi[a] = m->cfg.aabb[3 + a];
    p.inv[a] = m->cfg.inv_aabb_size[a];
    p.a_lo[a] = m->a_lo[a];
    p.a_inv[a] = m->a_inv[a];
  }
  p.near_t = m->cfg.near_t;
  p.far_t = m->cfg.far_t;
  p.step = m->cfg.step_size;
  p.a_thres = m->cfg.alpha_filter_thres;
  p.aD = m->aD;
  p.aH = m->aH;
  p.aW = m->aW;
  p.has_mask = m->alpha_bits != nullptr;
  p.a_bits = m->alpha_bits;
  p.a_coarse = m->alpha_coarse;
  p.a_full = m->alpha_full;
  p.cD = (m->aD + 3) / 4;
  p.cH = (m->aH + 3) / 4;
  p.cW = (m->aW + 3) / 4;
  p.S = S;
  p.words = (S + 31) / 32;
  p.kbits = gnr_sample_bits(S);
  p.mode = m->cfg.sampling_mode;
  p.hull_a = m->hull_near_term;
  p.hull_u = m->hull_u;
  return p;
}

int gnr_check_lattice(const GnrModel* m) {
  if (m->app_lattice && !m->app_lat_valid) {
    gnr_set_error("appearance planes, lines or MLP weights were uploaded after the appearance lattice was built: "
                  "call gnr_build_appearance_lattice again");
    return -1;
  }
  if (m->den_lattice && !m->lat_valid) {
    gnr_set_error("density planes or lines were uploaded after the density lattice was built: call gnr_build_density_lattice again");
    return -1;
  }
  return 0;
}

int gnr_check_sampler(const GnrModel* m, int S) {
  if (!m) {
    gnr_set_error("null model");
    return -1;
  }
  if (S < 1) {
    gnr_set_error("bad sample count %d", S);
    return -1;
  }
  // the hull sampler reads hull_near_term[k] and hull_u[k] for every k < S
  if (m->cfg.sampling_mode == 1 && (m->hull_samples != S || !m->hull_u || !m->hull_near_term)) {
    gnr_set_error("hull sampler: tables for %d samples per ray have not been uploaded (have %d)", S, m->hull_samples);
    return -1;
  }
  return 0;
}

int gnr_check_chunk(const GnrModel* m, int64_t n, int S, int64_t max_valid, int64_t max_app, const void* ws,
                    size_t ws_bytes) {
  if (!m) {
    gnr_set_error("null model");
    return -1;
  }
  if (n < 1 || S < 1 || max_valid < 0 || max_app < 0) {
    gnr_set_error("bad chunk arguments: n_rays %lld (at least 1) n_samples %d max_valid %lld max_app %lld", (long long)n, S,
                  (long long)max_valid, (long long)max_app);
    return -1;
  }
  const int kbits = gnr_sample_bits(S);
  if (kbits > 20 || n > ((int64_t)1 << (32 - kbits))) {
    gnr_set_error("chunk of %lld rays x %d samples does not fit the 32-bit sample ids (max %lld rays at this sample count)",
                  (long long)n, S, (long long)((int64_t)1 << (32 - kbits)));
    return -1;
  }
  if (n * (int64_t)S > 0x7fffffffLL || max_valid > 0x7fffffffLL || max_app > 0x7fffffffLL) {
    gnr_set_error("chunk too large: n_rays * n_samples and the capacities must stay below 2^31");
    return -1;
  }
  for (int i = 0; i < m->cfg.n_pairs; ++i) {
    if (!m->den[i].plane || !m->den[i].line || !m->app[i].plane || !m->app[i].line) {
      gnr_set_error("plane/line pair %d has not been uploaded", i);
      return -1;
    }
  }
  if (!m->mlp.w1t) {
    gnr_set_error("MLP weights have not been uploaded");
    return -1;
  }
  if (gnr_check_sampler(m, S)) return -1;
  if (gnr_check_lattice(m)) return -1;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, max_app);
  if (!ws || ws_bytes < L.total) {
    gnr_set_error("workspace too small: have %zu bytes, need %zu", ws_bytes, L.total);
    return -1;
  }
  if (((uintptr_t)ws & 255) != 0) {
    gnr_set_error("workspace must be 256-byte aligned");
    return -1;
  }
  return 0;
}

extern "C" int gnr_workspace_bytes(const GnrModel* m, int64_t n_rays, int n_samples, int64_t max_valid, int64_t max_app,
                                   size_t* bytes_h) {
  if (!m || !bytes_h || n_rays < 0 || n_samples < 1 || max_valid < 0 || max_app < 0) {
    gnr_set_error("gnr_workspace_bytes: bad argument");
    return -1;
  }
  *bytes_h = gnr_ws_layout(m, n_rays, n_samples, max_valid, max_app).total;
  return 0;
}

extern "C" int gnr_debug_wait(GnrModel* m, int expire, int wait_limit) {
  if (!m || wait_limit < 0) {
    gnr_set_error("gnr_debug_wait: bad argument");
    return -1;
  }
  m->debug_expire_wait = expire ? 1 : 0;
  m->debug_wait_limit = wait_limit;
  return 0;
}

extern "C" int gnr_debug_phase_cycles(GnrModel* m, int on, long long* cycles_h) {
  if (!m) {
    gnr_set_error("gnr_debug_phase_cycles: null model");
    return -1;
  }
  DeviceGuard g(m->device);
  if (on) {
    if (!m->debug_prof) GNR_CUDA_OK(cudaMalloc(&m->debug_prof, 64 * sizeof(long long)));
    GNR_CUDA_OK(cudaMemset(m->debug_prof, 0, 64 * sizeof(long long)));
    return 0;
  }
  if (m->debug_prof) {
    GNR_CUDA_OK(cudaDeviceSynchronize());
    if (cycles_h) GNR_CUDA_OK(cudaMemcpy(cycles_h, m->debug_prof, 64 * sizeof(long long), cudaMemcpyDeviceToHost));
    cudaFree(m->debug_prof);
    m->debug_prof = nullptr;
  }
  return 0;
}

extern "C" int gnr_read_status(const void* workspace, int32_t* status_h, void* stream) {
  if (!workspace || !status_h) {
    gnr_set_error("gnr_read_status: null argument");
    return -1;
  }
  GNR_CUDA_OK(cudaMemcpyAsync(status_h, workspace, GNR_ST_WORDS * sizeof(int32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  GNR_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
  return 0;
}

// ---------------------------------------------------------------------------------------------
// stages
// ---------------------------------------------------------------------------------------------
static int launch_sample(GnrModel* m, const GnrSampleParams& p, const float* rays, int64_t n, char* ws, const GnrWs& L,
                         int64_t max_valid, cudaStream_t st) {
  int e = launch_sample_mask(m, p, rays, n, ws, L, st);
  if (e) return e;
  return launch_sample_compact(m, p, n, ws, L, max_valid, 1, st);
}

static int launch_weights(GnrModel* m, const GnrSampleParams& p, int64_t n, char* ws, const GnrWs& L, int64_t max_valid,
                          int64_t max_app, cudaStream_t st) {
  int e = launch_weights_only(m, p, n, ws, L, max_valid, st);
  if (e) return e;
  return launch_app_compact(m, p, n, ws, L, max_valid, max_app, st);
}

static int copy_out(void* dst, const void* src, size_t bytes, cudaStream_t st) {
  if (!dst || bytes == 0) return 0;
  GNR_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st));
  return 0;
}

static int run_app_gather(GnrModel* m, const GnrSampleParams& p, const float* rays, int64_t n, char* ws, const GnrWs& L,
                          int64_t max_valid, int64_t max_app, cudaStream_t st) {
  (void)n;
  (void)max_valid;
  (void)max_app;
  const GnrCoords c = gnr_coords_app(rays, ws, L);
  if (gnr_tc_basis_fused(m)) {
    unsigned char* hi = (unsigned char*)(ws + L.app_prod);
    return launch_app_products(m, p, c, hi, hi + L.app_prod_image, L.app_prod_tile, m->cfg.mlp_mode == 1 ? 2 : 1, st);
  }
  return launch_app_gather(m, p, c, L.feat_stride, (float*)(ws + L.app_feat), st);
}

static int run_mlp(GnrModel* m, const GnrSampleParams& p, const float* rays, char* ws, const GnrWs& L, int write_features,
                   cudaStream_t st) {
  const GnrCoords c = gnr_coords_app(rays, ws, L);
  float* feat = (float*)(ws + L.app_feat);
  float* rgb = (float*)(ws + L.app_rgb);
  if (m->cfg.mlp_mode == 0) return launch_mlp_simt(m, p, c, L.feat_stride, feat, rgb, st);
  const unsigned char* hi = (const unsigned char*)(ws + L.app_prod);
  return launch_mlp_tc(m, p, c, L.feat_stride, feat, write_features ? feat : nullptr, hi, hi + L.app_prod_image,
                       L.app_prod_tile, rgb, (int32_t*)(ws + L.status), 0, st);
}

static int run_appearance(GnrModel* m, const GnrSampleParams& p, const float* rays, int64_t n, char* ws, const GnrWs& L,
                          int64_t max_valid, int64_t max_app, cudaStream_t st) {
  GNR_LAUNCH_OK(run_app_gather(m, p, rays, n, ws, L, max_valid, max_app, st));
  GNR_LAUNCH_OK(run_mlp(m, p, rays, ws, L, /*write_features=*/1, st));
  return 0;
}

extern "C" int gnr_sample(GnrModel* m, const float* rays, int64_t n, int S, void* workspace, size_t ws_bytes,
                          int64_t max_valid, float* t_min, int32_t* counts, int32_t* offsets, uint32_t* mask_words,
                          uint32_t* ids, void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, 0, workspace, ws_bytes);
  if (rc) return rc;
  if (!rays && n > 0) {
    gnr_set_error("gnr_sample: null rays");
    return -1;
  }
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, 0);
  GnrSampleParams p = gnr_sample_params(m, S);
  GNR_CUDA_OK(cudaMemsetAsync(ws + L.status, 0, GNR_ST_WORDS * sizeof(int32_t), st));
  GNR_LAUNCH_OK(launch_sample(m, p, rays, n, ws, L, max_valid, st));
  if (copy_out(t_min, ws + L.t_min, (size_t)n * 4, st)) return -2;
  if (copy_out(counts, ws + L.counts, (size_t)n * 4, st)) return -2;
  if (copy_out(offsets, ws + L.offsets, (size_t)(n + 1) * 4, st)) return -2;
  if (copy_out(mask_words, ws + L.words, (size_t)n * p.words * 4, st)) return -2;
  if (copy_out(ids, ws + L.ids, (size_t)max_valid * 4, st)) return -2;
  return 0;
}

extern "C" int gnr_density(GnrModel* m, const float* rays, int64_t n, int S, void* workspace, size_t ws_bytes,
                           int64_t max_valid, float* sigma_feature, float* sigma, void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, 0, workspace, ws_bytes);
  if (rc) return rc;
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, 0);
  GnrSampleParams p = gnr_sample_params(m, S);
  GNR_LAUNCH_OK(launch_density(m, p, gnr_coords_valid(rays, ws, L), (float*)(ws + L.sigma_feat), (float*)(ws + L.sigma), st));
  if (copy_out(sigma_feature, ws + L.sigma_feat, (size_t)max_valid * 4, st)) return -2;
  if (copy_out(sigma, ws + L.sigma, (size_t)max_valid * 4, st)) return -2;
  return 0;
}

extern "C" int gnr_march(GnrModel* m, const float* rays, int64_t n, int S, void* workspace, size_t ws_bytes,
                         int64_t max_valid, int64_t max_app, float* weights, float* acc, float* depth,
                         int32_t* app_counts, int32_t* app_offsets, int32_t* app_index, void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, max_app, workspace, ws_bytes);
  if (rc) return rc;
  if (!rays) {
    gnr_set_error("gnr_march: null rays");
    return -1;
  }
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, max_app);
  GnrSampleParams p = gnr_sample_params(m, S);
  // a caller that takes neither the per-sample weights nor the valid-list index of the entries gets the frame loop's
  // form: only the samples above the appearance threshold are written (the list, counts and offsets are the same)
  const int list_only = (weights == nullptr && app_index == nullptr) ? 1 : 0;
  GNR_LAUNCH_OK(launch_march(m, p, rays, n, ws, L, st, list_only));
  GNR_LAUNCH_OK(launch_app_compact(m, p, n, ws, L, max_valid, max_app, st, list_only));
  if (copy_out(weights, ws + L.weight, (size_t)max_valid * 4, st)) return -2;
  if (copy_out(acc, ws + L.acc, (size_t)n * 4, st)) return -2;
  if (copy_out(depth, ws + L.depth, (size_t)n * 4, st)) return -2;
  if (copy_out(app_counts, ws + L.app_counts, (size_t)n * 4, st)) return -2;
  if (copy_out(app_offsets, ws + L.app_offsets, (size_t)(n + 1) * 4, st)) return -2;
  if (copy_out(app_index, ws + L.app_index, (size_t)max_app * 4, st)) return -2;
  return 0;
}

extern "C" int gnr_weights(GnrModel* m, const float* rays, int64_t n, int S, void* workspace, size_t ws_bytes,
                           int64_t max_valid, int64_t max_app, float* weights, float* acc, float* depth,
                           int32_t* app_counts, int32_t* app_offsets, int32_t* app_index, void* stream) {
  (void)rays;
  int rc = gnr_check_chunk(m, n, S, max_valid, max_app, workspace, ws_bytes);
  if (rc) return rc;
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, max_app);
  GnrSampleParams p = gnr_sample_params(m, S);
  GNR_LAUNCH_OK(launch_weights(m, p, n, ws, L, max_valid, max_app, st));
  if (copy_out(weights, ws + L.weight, (size_t)max_valid * 4, st)) return -2;
  if (copy_out(acc, ws + L.acc, (size_t)n * 4, st)) return -2;
  if (copy_out(depth, ws + L.depth, (size_t)n * 4, st)) return -2;
  if (copy_out(app_counts, ws + L.app_counts, (size_t)n * 4, st)) return -2;
  if (copy_out(app_offsets, ws + L.app_offsets, (size_t)(n + 1) * 4, st)) return -2;
  if (copy_out(app_index, ws + L.app_index, (size_t)max_app * 4, st)) return -2;
  return 0;
}

extern "C" int gnr_appearance(GnrModel* m, const float* rays, int64_t n, int S, void* workspace, size_t ws_bytes,
                              int64_t max_valid, int64_t max_app, float* app_features, float* rgb, void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, max_app, workspace, ws_bytes);
  if (rc) return rc;
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, max_app);
  GnrSampleParams p = gnr_sample_params(m, S);
  rc = run_appearance(m, p, rays, n, ws, L, max_valid, max_app, st);
  if (rc) return rc;
  if (app_features) {
    GNR_CUDA_OK(cudaMemcpy2DAsync(app_features, (size_t)m->cfg.app_dim * 4, ws + L.app_feat, (size_t)L.feat_stride * 4,
                                  (size_t)m->cfg.app_dim * 4, (size_t)max_app, cudaMemcpyDeviceToDevice, st));
  }
  if (copy_out(rgb, ws + L.app_rgb, (size_t)max_app * 12, st)) return -2;
  return 0;
}

extern "C" int gnr_composite(GnrModel* m, int64_t n, int white_bg, void* workspace, size_t ws_bytes, int64_t max_valid,
                             int64_t max_app, int S, float* rgb_map, float* depth_map, void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, max_app, workspace, ws_bytes);
  if (rc) return rc;
  DeviceGuard g(m->device);
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, max_app);
  GNR_LAUNCH_OK(launch_composite(m, n, white_bg, ws, L, rgb_map, depth_map, (cudaStream_t)stream));
  return 0;
}

static int render_chunk_impl(GnrModel* m, const float* rays, int64_t n, int S, int white_bg, char* ws,
                             int64_t max_valid, int64_t max_app, float* rgb_map, float* depth_map, cudaStream_t st) {
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, max_app);
  GnrSampleParams p = gnr_sample_params(m, S);
  GNR_CUDA_OK(cudaMemsetAsync(ws + L.status, 0, GNR_ST_WORDS * sizeof(int32_t), st));
  {
    StageScope sc(m, GNR_STAGE_SAMPLE, 1, st);
    GNR_LAUNCH_OK(launch_sample_mask(m, p, rays, n, ws, L, st));
  }
  {
    const int fused = m->cfg.ert_transmittance >= 0.0f;
    StageScope sc(m, GNR_STAGE_COMPACT, fused ? 3 : 4, st);
    GNR_LAUNCH_OK(launch_sample_compact(m, p, n, ws, L, max_valid, fused ? 0 : 1, st));
  }
  if (m->cfg.ert_transmittance >= 0.0f) {
    // fused density + weights pass (with early ray termination when the threshold is > 0)
    StageScope sc(m, GNR_STAGE_DENSITY, 1, st);
    GNR_LAUNCH_OK(launch_march(m, p, rays, n, ws, L, st, /*list_only=*/1));
  } else {
    {
      StageScope sc(m, GNR_STAGE_DENSITY, 1, st);
      GNR_LAUNCH_OK(launch_density(m, p, gnr_coords_valid(rays, ws, L), (float*)(ws + L.sigma_feat), (float*)(ws + L.sigma), st));
    }
    {
      StageScope sc(m, GNR_STAGE_WEIGHTS, 1, st);
      GNR_LAUNCH_OK(launch_weights_only(m, p, n, ws, L, max_valid, st));
    }
  }
  {
    StageScope sc(m, GNR_STAGE_COMPACT_APP, 4, st);
    GNR_LAUNCH_OK(launch_app_compact(m, p, n, ws, L, max_valid, max_app, st, /*packed=*/m->cfg.ert_transmittance >= 0.0f ? 1 : 0));
  }
  if (gnr_app_fusable(m)) {
    // gather + basis projection + MLP as one kernel: no operand of a sample leaves the SM
    StageScope sc(m, GNR_STAGE_MLP, 1, st);
    if (m->cfg.unfused_appearance == 2 && !m->debug_prof)
      GNR_LAUNCH_OK(launch_app_mlp_stream(m, p, gnr_coords_app(rays, ws, L), (float*)(ws + L.app_rgb), (int32_t*)(ws + L.status), st));
    else
      GNR_LAUNCH_OK(launch_app_mlp_fused(m, p, gnr_coords_app(rays, ws, L), (float*)(ws + L.app_rgb), (int32_t*)(ws + L.status), st));
  } else {
    {
      StageScope sc(m, GNR_STAGE_APP_GATHER, 1, st);
      GNR_LAUNCH_OK(run_app_gather(m, p, rays, n, ws, L, max_valid, max_app, st));
    }
    {
      StageScope sc(m, GNR_STAGE_MLP, 1, st);
      GNR_LAUNCH_OK(run_mlp(m, p, rays, ws, L, /*write_features=*/0, st));
    }
  }
  {
    StageScope sc(m, GNR_STAGE_COMPOSITE, 1, st);
    GNR_LAUNCH_OK(launch_composite(m, n, white_bg, ws, L, rgb_map, depth_map, st));
  }
  return 0;
}

extern "C" int gnr_profile_enable(GnrModel* m, int on) {
  if (!m) {
    gnr_set_error("gnr_profile_enable: null model");
    return -1;
  }
  DeviceGuard g(m->device);
  if (on && !m->prof) m->prof = new (std::nothrow) GnrProfiler();
  if (!on && m->prof) {
    cudaDeviceSynchronize();
    delete m->prof;
    m->prof = nullptr;
  }
  return 0;
}

extern "C" int gnr_profile_collect(GnrModel* m, float* stage_ms_h, int64_t* launches_h) {
  if (!m || !stage_ms_h || !launches_h) {
    gnr_set_error("gnr_profile_collect: null argument");
    return -1;
  }
  if (!m->prof) {
    gnr_set_error("gnr_profile_collect: profiling is not enabled");
    return -1;
  }
  DeviceGuard g(m->device);
  for (auto& s : m->prof->spans) {
    GNR_CUDA_OK(cudaEventSynchronize(s.b));
    float ms = 0.0f;
    GNR_CUDA_OK(cudaEventElapsedTime(&ms, s.a, s.b));
    stage_ms_h[s.stage] += ms;
    launches_h[s.stage] += s.launches;
    m->prof->pool.push_back(s.a);
    m->prof->pool.push_back(s.b);
  }
  m->prof->spans.clear();
  return 0;
}

extern "C" int gnr_render_chunk(GnrModel* m, const float* rays, int64_t n, int S, int white_bg, void* workspace,
                                size_t ws_bytes, int64_t max_valid, int64_t max_app, float* rgb_map, float* depth_map,
                                void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, max_app, workspace, ws_bytes);
  if (rc) return rc;
  if (n == 0) return 0;
  if (!rays) {
    gnr_set_error("gnr_render_chunk: null rays");
    return -1;
  }
  DeviceGuard g(m->device);
  return render_chunk_impl(m, rays, n, S, white_bg, (char*)workspace, max_valid, max_app, rgb_map, depth_map,
                           (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// split-stage and point-mode entries (model-parallel renderers compose these with collectives)
// ---------------------------------------------------------------------------------------------
static GnrCoords coords_points(const float* xyz, const float* view, int64_t n, int stride = 3) {
  GnrCoords c;
  memset(&c, 0, sizeof(c));
  c.xyz_direct = xyz;
  c.view_direct = view;
  c.point_stride = stride;
  c.total_direct = n;
  c.capacity = n;
  return c;
}

struct PointScratch {
  size_t status, feat, prod, total, prod_image;
  int tile_bytes, terms;
};

static PointScratch point_scratch(const GnrModel* m, int64_t n) {
  PointScratch s;
  memset(&s, 0, sizeof(s));
  size_t off = 0;
  s.status = off;
  off = align_up(off + GNR_ST_WORDS * 4, 256);
  s.feat = off;
  off = align_up(off + (size_t)n * 28 * 4, 256);
  if (m->cfg.mlp_mode != 0 && gnr_tc_basis_fused(m)) {
    s.terms = m->cfg.mlp_mode == 1 ? 2 : 1;
    s.tile_bytes = gnr_tc_tile_bytes(m);
    s.prod_image = align_up((size_t)((n + 127) / 128) * s.tile_bytes, 256);
    s.prod = off;
    off += s.prod_image * s.terms;
  }
  s.total = off;
  return s;
}

static int check_points(const GnrModel* m, const char* who, int64_t n, const void* scratch, size_t scratch_bytes) {
  if (!m) {
    gnr_set_error("%s: null model", who);
    return -1;
  }
  if (n < 0 || n > 0x7fffffffLL) {
    gnr_set_error("%s: bad point count %lld", who, (long long)n);
    return -1;
  }
  if (!m->mlp.w1t || !m->app[0].plane || !m->den[0].plane) {
    gnr_set_error("%s: model parameters have not been uploaded", who);
    return -1;
  }
  if (gnr_check_lattice(m)) return -1;
  if (scratch_bytes != (size_t)-1) {
    const PointScratch s = point_scratch(m, n);
    if (!scratch || scratch_bytes < s.total || ((uintptr_t)scratch & 255) != 0) {
      gnr_set_error("%s: scratch must be 256-byte aligned and hold %zu bytes (got %zu)", who, s.total, scratch_bytes);
      return -1;
    }
  }
  return 0;
}

extern "C" int gnr_points_scratch_bytes(const GnrModel* m, int64_t n, size_t* bytes_h) {
  if (!m || !bytes_h || n < 0) {
    gnr_set_error("gnr_points_scratch_bytes: bad argument");
    return -1;
  }
  *bytes_h = point_scratch(m, n).total;
  return 0;
}

extern "C" int gnr_density_points(GnrModel* m, const float* xyz, int64_t n, float* sigma_feature, float* sigma, void* stream) {
  int rc = check_points(m, "gnr_density_points", n, nullptr, (size_t)-1);
  if (rc) return rc;
  if (n == 0) return 0;
  if (!xyz || !sigma) {
    gnr_set_error("gnr_density_points: null xyz or sigma");
    return -1;
  }
  DeviceGuard g(m->device);
  GnrSampleParams p = gnr_sample_params(m, 1);
  GNR_LAUNCH_OK(launch_density(m, p, coords_points(xyz, nullptr, n), sigma_feature, sigma, (cudaStream_t)stream));
  return 0;
}

static int mlp_points(GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, char* sc, const PointScratch& S, int fused,
                      float* feat_copy, float* rgb, cudaStream_t st) {
  float* feat = (float*)(sc + S.feat);
  if (m->cfg.mlp_mode == 0) {
    GNR_LAUNCH_OK(launch_mlp_simt(m, p, c, 28, feat, rgb, st));
  } else {
    const unsigned char* hi = (const unsigned char*)(sc + S.prod);
    GNR_LAUNCH_OK(launch_mlp_tc(m, p, c, 28, feat, (fused && feat_copy) ? feat : nullptr, hi, hi + S.prod_image, S.tile_bytes, rgb,
                                (int32_t*)(sc + S.status), fused ? 0 : 1, st));
  }
  if (feat_copy) {
    GNR_CUDA_OK(cudaMemcpy2DAsync(feat_copy, (size_t)m->cfg.app_dim * 4, feat, 28 * 4, (size_t)m->cfg.app_dim * 4,
                                  (size_t)c.total_direct, cudaMemcpyDeviceToDevice, st));
  }
  return 0;
}

static int appearance_points_impl(GnrModel* m, const GnrCoords& c, int64_t n, void* scratch, float* features, float* rgb,
                                  void* stream);

extern "C" int gnr_appearance_points(GnrModel* m, const float* xyz, const float* view, int64_t n, void* scratch,
                                     size_t scratch_bytes, float* features, float* rgb, void* stream) {
  int rc = check_points(m, "gnr_appearance_points", n, scratch, scratch_bytes);
  if (rc) return rc;
  if (n == 0) return 0;
  if (!xyz || !view || !rgb) {
    gnr_set_error("gnr_appearance_points: null xyz, view or rgb");
    return -1;
  }
  return appearance_points_impl(m, coords_points(xyz, view, n), n, scratch, features, rgb, stream);
}

extern "C" int gnr_appearance_rows(GnrModel* m, const float* rows, int64_t n, void* scratch, size_t scratch_bytes, float* rgb,
                                   void* stream) {
  int rc = check_points(m, "gnr_appearance_rows", n, scratch, scratch_bytes);
  if (rc) return rc;
  if (n == 0) return 0;
  if (!rows || !rgb) {
    gnr_set_error("gnr_appearance_rows: null rows or rgb");
    return -1;
  }
  return appearance_points_impl(m, coords_points(rows, rows + 3, n, 6), n, scratch, nullptr, rgb, stream);
}

static int appearance_points_impl(GnrModel* m, const GnrCoords& c, int64_t n, void* scratch, float* features, float* rgb,
                                  void* stream) {
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* sc = (char*)scratch;
  const PointScratch S = point_scratch(m, n);
  GnrSampleParams p = gnr_sample_params(m, 1);
  GNR_CUDA_OK(cudaMemsetAsync(sc + S.status, 0, GNR_ST_WORDS * 4, st));
  if (!features && gnr_app_fusable(m)) {
    // gather + basis projection + MLP as one kernel, the points' operands never leaving the SM
    GNR_LAUNCH_OK(launch_app_mlp_fused(m, p, c, rgb, (int32_t*)(sc + S.status), st));
    return 0;
  }
  const int fused = m->cfg.mlp_mode != 0 && gnr_tc_basis_fused(m);
  if (fused) {
    unsigned char* hi = (unsigned char*)(sc + S.prod);
    GNR_LAUNCH_OK(launch_app_products(m, p, c, hi, hi + S.prod_image, S.tile_bytes, S.terms, st));
  } else {
    GNR_LAUNCH_OK(launch_app_gather(m, p, c, 28, (float*)(sc + S.feat), st));
  }
  return mlp_points(m, p, c, sc, S, fused, features, rgb, st);
}

extern "C" int gnr_app_features_points(GnrModel* m, const float* xyz, int64_t n, void* scratch, size_t scratch_bytes,
                                       float* features, void* stream) {
  int rc = check_points(m, "gnr_app_features_points", n, scratch, scratch_bytes);
  if (rc) return rc;
  if (n == 0) return 0;
  if (!xyz || !features) {
    gnr_set_error("gnr_app_features_points: null xyz or features");
    return -1;
  }
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* sc = (char*)scratch;
  const PointScratch S = point_scratch(m, n);
  GnrSampleParams p = gnr_sample_params(m, 1);
  const GnrCoords c = coords_points(xyz, nullptr, n);
  float* feat = (float*)(sc + S.feat);
  if (m->cfg.mlp_mode != 0 && gnr_tc_basis_fused(m)) {
    // product tiles, then the projection alone on the tensor cores (fp32 accumulate)
    GNR_CUDA_OK(cudaMemsetAsync(sc + S.status, 0, GNR_ST_WORDS * 4, st));
    unsigned char* hi = (unsigned char*)(sc + S.prod);
    GNR_LAUNCH_OK(launch_app_products(m, p, c, hi, hi + S.prod_image, S.tile_bytes, S.terms, st));
    GNR_LAUNCH_OK(launch_mlp_tc(m, p, c, 28, nullptr, feat, hi, hi + S.prod_image, S.tile_bytes, nullptr, (int32_t*)(sc + S.status), 0, st,
                                /*basis_only=*/1));
  } else {
    GNR_LAUNCH_OK(launch_app_gather(m, p, c, 28, feat, st));
  }
  GNR_CUDA_OK(cudaMemcpy2DAsync(features, (size_t)m->cfg.app_dim * 4, feat, 28 * 4, (size_t)m->cfg.app_dim * 4, (size_t)n,
                                cudaMemcpyDeviceToDevice, st));
  return 0;
}

extern "C" int gnr_project_slice_points(GnrModel* m, const float* xyz, int point_stride, int64_t n, void* features_h,
                                        int32_t* status, void* stream) {
  int rc = check_points(m, "gnr_project_slice_points", n, nullptr, (size_t)-1);
  if (rc) return rc;
  if (n == 0) return 0;
  if (!xyz || !features_h || !status || point_stride < 3) {
    gnr_set_error("gnr_project_slice_points: null xyz, features or status, or a point stride below 3");
    return -1;
  }
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  GNR_CUDA_OK(cudaMemsetAsync(status, 0, GNR_ST_WORDS * 4, st));
  GNR_LAUNCH_OK(launch_app_slice_project(m, xyz, point_stride, n, features_h, status, st));
  return 0;
}

extern "C" int gnr_sum_partials(GnrModel* m, const void* parts_h, int n_parts, int64_t rows, int64_t part_stride_rows,
                                float* features, void* stream) {
  if (!m || !parts_h || !features || n_parts < 1 || rows < 0 || part_stride_rows < rows) {
    gnr_set_error("gnr_sum_partials: null model, parts or features, or bad sizes (%d parts, %lld rows, stride %lld)", n_parts,
                  (long long)rows, (long long)part_stride_rows);
    return -1;
  }
  DeviceGuard g(m->device);
  GNR_LAUNCH_OK(launch_sum_partials(parts_h, n_parts, rows, part_stride_rows, m->cfg.app_dim, m->cfg.app_dim, features,
                                    (cudaStream_t)stream));
  return 0;
}

extern "C" int gnr_mlp_partial_rows(GnrModel* m, const void* parts_h, int n_parts, int64_t part_stride_rows,
                                    const float* rows6, int64_t n, void* scratch, size_t scratch_bytes, float* rgb,
                                    void* stream) {
  int rc = check_points(m, "gnr_mlp_partial_rows", n, scratch, scratch_bytes);
  if (rc) return rc;
  if (n == 0) return 0;
  if (!parts_h || !rows6 || !rgb || n_parts < 1 || part_stride_rows < n) {
    gnr_set_error("gnr_mlp_partial_rows: null parts, rows or rgb, or bad sizes (%d parts, stride %lld, %lld rows)", n_parts,
                  (long long)part_stride_rows, (long long)n);
    return -1;
  }
  if (m->cfg.mlp_mode != 2 || m->cfg.unfused_appearance == 1 || !m->mlp.tc_image) {
    gnr_set_error("gnr_mlp_partial_rows: needs mlp_mode 2 and the one-kernel appearance path");
    return -1;
  }
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* sc = (char*)scratch;
  const PointScratch S = point_scratch(m, n);
  GnrSampleParams p = gnr_sample_params(m, 1);
  GNR_CUDA_OK(cudaMemsetAsync(sc + S.status, 0, GNR_ST_WORDS * 4, st));
  // view directions are columns 3..5 of the (point, view) rows the appearance list was routed as
  GNR_LAUNCH_OK(launch_app_mlp_fused(m, p, coords_points(nullptr, rows6 + 3, n, 6), rgb, (int32_t*)(sc + S.status), st, nullptr, 0,
                                     parts_h, n_parts, part_stride_rows));
  return 0;
}

extern "C" int gnr_mlp_features(GnrModel* m, const float* features, const float* view, int64_t n, void* scratch,
                                size_t scratch_bytes, float* rgb, void* stream) {
  int rc = check_points(m, "gnr_mlp_features", n, scratch, scratch_bytes);
  if (rc) return rc;
  if (n == 0) return 0;
  if (!features || !view || !rgb) {
    gnr_set_error("gnr_mlp_features: null features, view or rgb");
    return -1;
  }
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* sc = (char*)scratch;
  const PointScratch S = point_scratch(m, n);
  GnrSampleParams p = gnr_sample_params(m, 1);
  GNR_CUDA_OK(cudaMemsetAsync(sc + S.status, 0, GNR_ST_WORDS * 4, st));
  if (m->cfg.mlp_mode == 2 && m->cfg.unfused_appearance != 1 && m->mlp.tc_image) {
    // positional encoding + the three layers in the one-kernel form, features read in place
    GNR_LAUNCH_OK(launch_app_mlp_fused(m, p, coords_points(nullptr, view, n), rgb, (int32_t*)(sc + S.status), st, features,
                                       m->cfg.app_dim));
    return 0;
  }
  GNR_CUDA_OK(cudaMemsetAsync(sc + S.feat, 0, (size_t)n * 28 * 4, st));
  GNR_CUDA_OK(cudaMemcpy2DAsync(sc + S.feat, 28 * 4, features, (size_t)m->cfg.app_dim * 4, (size_t)m->cfg.app_dim * 4, (size_t)n,
                                cudaMemcpyDeviceToDevice, st));
  return mlp_points(m, p, coords_points(nullptr, view, n), sc, S, /*fused=*/0, nullptr, rgb, st);
}

extern "C" int gnr_valid_positions(GnrModel* m, const float* rays, int64_t n, int S, void* workspace, size_t ws_bytes,
                                   int64_t max_valid, float* xyz, int32_t* ray_index, void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, 0, workspace, ws_bytes);
  if (rc) return rc;
  if (!rays || !xyz) {
    gnr_set_error("gnr_valid_positions: null rays or xyz");
    return -1;
  }
  DeviceGuard g(m->device);
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, 0);
  GnrSampleParams p = gnr_sample_params(m, S);
  GNR_LAUNCH_OK(launch_positions(m, p, gnr_coords_valid(rays, ws, L), xyz, ray_index, (cudaStream_t)stream));
  return 0;
}

extern "C" int gnr_route_blocks(GnrModel* m, const float* rays, int64_t n, int S, void* workspace, size_t ws_bytes,
                                int64_t max_valid, int64_t max_app, int which_list, int px, int py, float* send_points,
                                int32_t* dest_row, int32_t* counts, int32_t* block_of, void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, max_app, workspace, ws_bytes);
  if (rc) return rc;
  if (!rays || !send_points || !dest_row || !counts || (which_list != 0 && which_list != 1)) {
    gnr_set_error("gnr_route_blocks: null rays / send_points / dest_row / counts, or which_list not 0 (valid) / 1 (appearance)");
    return -1;
  }
  DeviceGuard g(m->device);
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, max_app);
  GnrSampleParams p = gnr_sample_params(m, S);
  const GnrCoords c = which_list == 0 ? gnr_coords_valid(rays, ws, L) : gnr_coords_app(rays, ws, L);
  GNR_LAUNCH_OK(launch_route_blocks(m, p, c, px, py, which_list == 1, send_points, dest_row, counts, block_of, (cudaStream_t)stream));
  return 0;
}

extern "C" int gnr_query_one_kernel_appearance(const GnrModel* m) { return m ? gnr_app_fusable(m) : 0; }

extern "C" int gnr_route_block_ids(GnrModel* m, const float* rays, int64_t n, int S, void* workspace, size_t ws_bytes,
                                   int64_t max_valid, int64_t max_app, int which_list, int px, int py, uint32_t ray_base,
                                   uint32_t* send_ids, int32_t* dest_row, int32_t* counts, void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, max_app, workspace, ws_bytes);
  if (rc) return rc;
  if (!rays || !send_ids || !dest_row || !counts || (which_list != 0 && which_list != 1)) {
    gnr_set_error("gnr_route_block_ids: null rays / send_ids / dest_row / counts, or which_list not 0 (valid) / 1 (appearance)");
    return -1;
  }
  const int kbits = gnr_sample_bits(S);
  if (((uint64_t)ray_base + (uint64_t)n) >> (32 - kbits)) {
    gnr_set_error("gnr_route_block_ids: ray number %llu does not fit the %d bits an id leaves for it",
                  (unsigned long long)ray_base + (unsigned long long)n, 32 - kbits);
    return -1;
  }
  DeviceGuard g(m->device);
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, max_app);
  GnrSampleParams p = gnr_sample_params(m, S);
  const GnrCoords c = which_list == 0 ? gnr_coords_valid(rays, ws, L) : gnr_coords_app(rays, ws, L);
  GNR_LAUNCH_OK(launch_route_blocks(m, p, c, px, py, 2, (float*)send_ids, dest_row, counts, nullptr, (cudaStream_t)stream, ray_base));
  return 0;
}

// list-mode coordinates at a block owner: ids that carry ray numbers of the gathered ray table, the sampler's global
// box in `p`, positions expressed in block `block` of a px x py division
static int coords_owner_list(const char* who, const GnrModel* owner, const GnrModel* sampler, const float* rays_all,
                             const float* t_min_all, const uint32_t* ids, int64_t n, int px, int py, int block, GnrCoords* c) {
  if (!owner || !sampler || !rays_all || !t_min_all || !ids || n < 0 || n > 0x7fffffffLL) {
    gnr_set_error("%s: null model, rays, t_min or ids, or a bad count", who);
    return -1;
  }
  if (px < 1 || py < 1 || block < 0 || block >= px * py) {
    gnr_set_error("%s: block %d is not one of %d x %d", who, block, px, py);
    return -1;
  }
  if (owner->device != sampler->device) {
    gnr_set_error("%s: sampler and owner live on different devices", who);
    return -1;
  }
  memset(c, 0, sizeof(*c));
  c->rays = rays_all;
  c->t_min = t_min_all;
  c->ids = ids;
  c->point_stride = 3;
  c->total_direct = n;
  c->capacity = n;
  c->blk_px = px;
  c->blk_py = py;
  c->blk_bx = block / py;
  c->blk_by = block % py;
  c->blk_pw = (float)(2.0 / px);
  c->blk_ph = (float)(2.0 / py);
  return 0;
}

extern "C" int gnr_density_list(GnrModel* owner, const GnrModel* sampler, const float* rays_all, const float* t_min_all,
                                const uint32_t* ids, int64_t n, int S, int px, int py, int block, float* sigma, void* stream) {
  GnrCoords c;
  int rc = coords_owner_list("gnr_density_list", owner, sampler, rays_all, t_min_all, ids, n, px, py, block, &c);
  if (rc) return rc;
  rc = check_points(owner, "gnr_density_list", n, nullptr, (size_t)-1);
  if (rc) return rc;
  if (n == 0) return 0;
  if (!sigma) {
    gnr_set_error("gnr_density_list: null sigma");
    return -1;
  }
  DeviceGuard g(owner->device);
  const GnrSampleParams p = gnr_sample_params(sampler, S);  // the ray parametrisation and the global box are the sampler's
  GNR_LAUNCH_OK(launch_density(owner, p, c, nullptr, sigma, (cudaStream_t)stream));
  return 0;
}

extern "C" int gnr_appearance_list(GnrModel* owner, const GnrModel* sampler, const float* rays_all, const float* t_min_all,
                                   const uint32_t* ids, int64_t n, int S, int px, int py, int block, void* scratch,
                                   size_t scratch_bytes, float* rgb, void* stream) {
  GnrCoords c;
  int rc = coords_owner_list("gnr_appearance_list", owner, sampler, rays_all, t_min_all, ids, n, px, py, block, &c);
  if (rc) return rc;
  rc = check_points(owner, "gnr_appearance_list", n, scratch, scratch_bytes);
  if (rc) return rc;
  if (n == 0) return 0;
  if (!rgb) {
    gnr_set_error("gnr_appearance_list: null rgb");
    return -1;
  }
  if (!gnr_app_fusable(owner)) {
    gnr_set_error("gnr_appearance_list: needs the one-kernel appearance path (mlp_mode 2, fp16 appearance planes of 48 channels)");
    return -1;
  }
  DeviceGuard g(owner->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* sc = (char*)scratch;
  const PointScratch Sc = point_scratch(owner, n);
  const GnrSampleParams p = gnr_sample_params(sampler, S);
  GNR_CUDA_OK(cudaMemsetAsync(sc + Sc.status, 0, GNR_ST_WORDS * 4, st));
  GNR_LAUNCH_OK(launch_app_mlp_fused(owner, p, c, rgb, (int32_t*)(sc + Sc.status), st));
  return 0;
}

extern "C" int gnr_weights_from_sigma(GnrModel* m, int64_t n, int S, void* workspace, size_t ws_bytes, int64_t max_valid,
                                      int64_t max_app, const float* sigma_in, int32_t* app_index, void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, max_app, workspace, ws_bytes);
  if (rc) return rc;
  if (!sigma_in) {
    gnr_set_error("gnr_weights_from_sigma: null sigma");
    return -1;
  }
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, max_app);
  GnrSampleParams p = gnr_sample_params(m, S);
  GNR_CUDA_OK(cudaMemcpyAsync(ws + L.sigma, sigma_in, (size_t)max_valid * 4, cudaMemcpyDeviceToDevice, st));
  GNR_LAUNCH_OK(launch_weights(m, p, n, ws, L, max_valid, max_app, st));
  if (copy_out(app_index, ws + L.app_index, (size_t)max_app * 4, st)) return -2;
  return 0;
}

extern "C" int gnr_weights_from_rows(GnrModel* m, int64_t n, int S, void* workspace, size_t ws_bytes, int64_t max_valid,
                                     int64_t max_app, const float* sigma_rows, const int32_t* rows, void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, max_app, workspace, ws_bytes);
  if (rc) return rc;
  if (!sigma_rows || !rows) {
    gnr_set_error("gnr_weights_from_rows: null sigma_rows or rows");
    return -1;
  }
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, max_app);
  GnrSampleParams p = gnr_sample_params(m, S);
  GNR_LAUNCH_OK(launch_weights_only(m, p, n, ws, L, max_valid, st, sigma_rows, rows));
  GNR_LAUNCH_OK(launch_app_compact(m, p, n, ws, L, max_valid, max_app, st, /*packed=*/1));
  return 0;
}

extern "C" int gnr_app_features(GnrModel* m, const float* rays, int64_t n, int S, void* workspace, size_t ws_bytes,
                                int64_t max_valid, int64_t max_app, float* features, int64_t n_features, void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, max_app, workspace, ws_bytes);
  if (rc) return rc;
  if (!rays || !features || n_features > max_app) {
    gnr_set_error("gnr_app_features: null rays or features, or more rows asked for than the list can hold");
    return -1;
  }
  const int64_t rows = n_features < 0 ? max_app : n_features;
  if (rows == 0) return 0;
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, max_app);
  GnrSampleParams p = gnr_sample_params(m, S);
  const GnrCoords c = gnr_coords_app(rays, ws, L);
  if (gnr_tc_basis_fused(m)) {
    // tensor-core path: fp16 product tiles, then the projection alone (tcgen05, fp32 accumulate)
    unsigned char* hi = (unsigned char*)(ws + L.app_prod);
    GNR_LAUNCH_OK(launch_app_products(m, p, c, hi, hi + L.app_prod_image, L.app_prod_tile, m->cfg.mlp_mode == 1 ? 2 : 1, st));
    GNR_LAUNCH_OK(launch_mlp_tc(m, p, c, L.feat_stride, nullptr, (float*)(ws + L.app_feat), hi, hi + L.app_prod_image,
                                L.app_prod_tile, (float*)(ws + L.app_rgb), (int32_t*)(ws + L.status), 0, st, /*basis_only=*/1));
  } else {
    GNR_LAUNCH_OK(launch_app_gather(m, p, c, L.feat_stride, (float*)(ws + L.app_feat), st));
  }
  GNR_CUDA_OK(cudaMemcpy2DAsync(features, (size_t)m->cfg.app_dim * 4, ws + L.app_feat, (size_t)L.feat_stride * 4,
                                (size_t)m->cfg.app_dim * 4, (size_t)rows, cudaMemcpyDeviceToDevice, st));
  return 0;
}

extern "C" int gnr_composite_rgb(GnrModel* m, int64_t n, int white_bg, void* workspace, size_t ws_bytes, int64_t max_valid,
                                 int64_t max_app, int S, const float* rgb_samples, int64_t n_samples_rgb, float* rgb_map,
                                 float* depth_map, void* stream) {
  int rc = gnr_check_chunk(m, n, S, max_valid, max_app, workspace, ws_bytes);
  if (rc) return rc;
  if (n_samples_rgb < 0 || n_samples_rgb > max_app || (!rgb_samples && n_samples_rgb > 0)) {
    gnr_set_error("gnr_composite_rgb: %lld colours do not fit the appearance list (capacity %lld)", (long long)n_samples_rgb,
                  (long long)max_app);
    return -1;
  }
  DeviceGuard g(m->device);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  GnrWs L = gnr_ws_layout(m, n, S, max_valid, max_app);
  if (n_samples_rgb > 0)
    GNR_CUDA_OK(cudaMemcpyAsync(ws + L.app_rgb, rgb_samples, (size_t)n_samples_rgb * 12, cudaMemcpyDeviceToDevice, st));
  GNR_LAUNCH_OK(launch_composite(m, n, white_bg, ws, L, rgb_map, depth_map, st));
  return 0;
}

// ---------------------------------------------------------------------------------------------
// host-buffer forward: two chunks in flight on two streams so that the copies of one chunk
// overlap the kernels of the other.
// ---------------------------------------------------------------------------------------------
extern "C" int gnr_render_host(GnrModel* m, const float* rays_h, int64_t n_rays, int S, int white_bg, int64_t chunk,
                               int64_t max_valid, int64_t max_app, float* rgb_h, float* depth_h, int32_t* status_h) {
  if (!m || !rays_h || n_rays < 0 || chunk < 1 || (!rgb_h && !depth_h)) {
    gnr_set_error("gnr_render_host: bad argument");
    return -1;
  }
  DeviceGuard g(m->device);
  if (chunk > n_rays && n_rays > 0) chunk = n_rays;
  GnrWs L = gnr_ws_layout(m, chunk, S, max_valid, max_app);
  const size_t ws_one = align_up(L.total, 256);
  if (m->host_chunk != chunk || m->host_ws_bytes < 2 * ws_one) {
    cudaDeviceSynchronize();
    free_dev(m->host_ws);
    free_dev(m->host_rays);
    free_dev(m->host_rgb);
    free_dev(m->host_depth);
    m->host_ws = nullptr;
    m->host_rays = m->host_rgb = m->host_depth = nullptr;
    m->host_ws_bytes = 0;
    m->host_chunk = 0;
    GNR_CUDA_OK(cudaMalloc(&m->host_ws, 2 * ws_one));
    GNR_CUDA_OK(cudaMalloc(&m->host_rays, 2 * (size_t)chunk * 6 * 4));
    GNR_CUDA_OK(cudaMalloc(&m->host_rgb, 2 * (size_t)chunk * 3 * 4));
    GNR_CUDA_OK(cudaMalloc(&m->host_depth, 2 * (size_t)chunk * 4));
    m->host_ws_bytes = 2 * ws_one;
    m->host_chunk = chunk;
  }
  for (int i = 0; i < 2; ++i) {
    if (!m->host_streams[i]) GNR_CUDA_OK(cudaStreamCreateWithFlags(&m->host_streams[i], cudaStreamNonBlocking));
  }
  int rc = gnr_check_chunk(m, chunk, S, max_valid, max_app, m->host_ws, ws_one);
  if (rc) return rc;
  const int64_t n_chunks = (n_rays + chunk - 1) / chunk;
  if (n_chunks > m->host_status_slots) {
    if (m->host_status) cudaFreeHost(m->host_status);
    m->host_status = nullptr;
    m->host_status_slots = 0;
    GNR_CUDA_OK(cudaMallocHost(&m->host_status, (size_t)n_chunks * GNR_ST_WORDS * sizeof(int32_t)));
    m->host_status_slots = n_chunks;
  }
  int32_t* st_all = m->host_status;  // pinned, so the status copies stay asynchronous
  for (int64_t c = 0; c < n_chunks; ++c) {
    const int b = (int)(c & 1);
    cudaStream_t st = m->host_streams[b];
    const int64_t first = c * chunk, n = (first + chunk <= n_rays) ? chunk : n_rays - first;
    char* ws = (char*)m->host_ws + b * ws_one;
    float* d_rays = m->host_rays + (size_t)b * chunk * 6;
    float* d_rgb = m->host_rgb + (size_t)b * chunk * 3;
    float* d_depth = m->host_depth + (size_t)b * chunk;
    GNR_CUDA_OK(cudaMemcpyAsync(d_rays, rays_h + first * 6, (size_t)n * 24, cudaMemcpyHostToDevice, st));
    rc = render_chunk_impl(m, d_rays, n, S, white_bg, ws, max_valid, max_app, d_rgb, d_depth, st);
    if (rc) return rc;
    if (rgb_h) GNR_CUDA_OK(cudaMemcpyAsync(rgb_h + first * 3, d_rgb, (size_t)n * 12, cudaMemcpyDeviceToHost, st));
    if (depth_h) GNR_CUDA_OK(cudaMemcpyAsync(depth_h + first, d_depth, (size_t)n * 4, cudaMemcpyDeviceToHost, st));
    GNR_CUDA_OK(cudaMemcpyAsync(&st_all[(size_t)c * GNR_ST_WORDS], ws, GNR_ST_WORDS * 4, cudaMemcpyDeviceToHost, st));
  }
  GNR_CUDA_OK(cudaStreamSynchronize(m->host_streams[0]));
  GNR_CUDA_OK(cudaStreamSynchronize(m->host_streams[1]));
  if (status_h) {
    for (int i = 0; i < GNR_ST_WORDS; ++i) status_h[i] = 0;
    for (int64_t c = 0; c < n_chunks; ++c) {
      const int32_t* s = &st_all[(size_t)c * GNR_ST_WORDS];
      status_h[GNR_ST_OVERFLOW_VALID] |= s[GNR_ST_OVERFLOW_VALID];
      status_h[GNR_ST_OVERFLOW_APP] |= s[GNR_ST_OVERFLOW_APP];
      status_h[GNR_ST_WAIT_EXPIRED] |= s[GNR_ST_WAIT_EXPIRED];
      // totals saturate instead of wrapping
      long long v = (long long)status_h[GNR_ST_NUM_VALID] + s[GNR_ST_NUM_VALID];
      long long a = (long long)status_h[GNR_ST_NUM_APP] + s[GNR_ST_NUM_APP];
      long long dn = (long long)status_h[GNR_ST_NUM_DENSITY] + s[GNR_ST_NUM_DENSITY];
      status_h[GNR_ST_NUM_DENSITY] = dn > 0x7fffffffLL ? 0x7fffffff : (int32_t)dn;
      status_h[GNR_ST_NUM_VALID] = v > 0x7fffffffLL ? 0x7fffffff : (int32_t)v;
      status_h[GNR_ST_NUM_APP] = a > 0x7fffffffLL ? 0x7fffffff : (int32_t)a;
    }
  }
  return 0;
}
