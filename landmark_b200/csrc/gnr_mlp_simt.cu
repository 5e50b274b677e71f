// Appearance MLP on the CUDA cores in fp32 (the reference-precision path).
//
// MLPRender_Fea.forward (app/models/mlp_render_fea.py:44-68) with positional_encoding
// (app/tools/utils.py:42-48): input = [feat, view, sin(feat 2^f), cos(feat 2^f),
// sin(view 2^f), cos(view 2^f)] -> Linear+ReLU -> Linear+ReLU -> Linear -> sigmoid.
// One persistent block per SM keeps all weights in shared memory and walks tiles of 64
// appearance samples; each thread owns a 4 (samples) x 8 (units) register tile.
#include "gnr_internal.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int TM = 64;    // samples per tile
constexpr int HID = 128;  // hidden width

struct MlpDims {
  int app_dim, fea_pe, view_pe, in_dim, k1_pad, feat_stride;
};

template <int K_IS_HID>
__device__ __forceinline__ void dense_relu(const float* __restrict__ wt, const float* __restrict__ bias,
                                           const float* __restrict__ xin, float* __restrict__ xout, int K) {
  // xin [K][TM], wt [K][HID], xout [HID][TM]
  const int tn = threadIdx.x & 15, tm = threadIdx.x >> 4;
  const int m0 = tm * 4, n0 = tn * 4;
  float acc[4][8];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[a][b] = 0.0f;
  const int kk = K_IS_HID ? HID : K;
#pragma unroll 4
  for (int k = 0; k < kk; ++k) {
    const float4 xv = *reinterpret_cast<const float4*>(xin + k * TM + m0);
    const float4 w0 = *reinterpret_cast<const float4*>(wt + k * HID + n0);
    const float4 w1 = *reinterpret_cast<const float4*>(wt + k * HID + 64 + n0);
    const float x[4] = {xv.x, xv.y, xv.z, xv.w};
    const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 8; ++b) acc[a][b] = fmaf(x[a], w[b], acc[a][b]);
  }
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    const int n = (b < 4) ? (n0 + b) : (64 + n0 + b - 4);
    const float bv = bias[n];
    float4 o;
    o.x = fmaxf(acc[0][b] + bv, 0.0f);
    o.y = fmaxf(acc[1][b] + bv, 0.0f);
    o.z = fmaxf(acc[2][b] + bv, 0.0f);
    o.w = fmaxf(acc[3][b] + bv, 0.0f);
    *reinterpret_cast<float4*>(xout + n * TM + m0) = o;
  }
}

__global__ void __launch_bounds__(kThreads, 1)
mlp_simt_kernel(MlpDims d, int kbits, GnrCoords crd, const float* __restrict__ feat, const float* __restrict__ g_w1t,
                const float* __restrict__ g_w2t,
                const float* __restrict__ g_w3, const float* __restrict__ g_b1, const float* __restrict__ g_b2,
                const float* __restrict__ g_b3, float* __restrict__ rgb_out) {
  extern __shared__ float4 smem_f4[];
  float* sm = reinterpret_cast<float*>(smem_f4);
  float* w1t = sm;                       // [k1_pad][HID]
  float* w2t = w1t + d.k1_pad * HID;     // [HID][HID]
  float* w3 = w2t + HID * HID;           // [3][HID]
  float* b1 = w3 + 3 * HID;              // [HID]
  float* b2 = b1 + HID;                  // [HID]
  float* b3 = b2 + HID;                  // [4]
  float* xa = b3 + 4;                    // [k1_pad][TM]   input tile, later layer-2 output
  float* xb = xa + d.k1_pad * TM;        // [HID][TM]      layer-1 output

  for (int i = threadIdx.x; i < d.k1_pad * HID; i += kThreads) w1t[i] = g_w1t[i];
  for (int i = threadIdx.x; i < HID * HID; i += kThreads) w2t[i] = g_w2t[i];
  for (int i = threadIdx.x; i < 3 * HID; i += kThreads) w3[i] = g_w3[i];
  for (int i = threadIdx.x; i < HID; i += kThreads) {
    b1[i] = g_b1[i];
    b2[i] = g_b2[i];
  }
  if (threadIdx.x < 4) b3[threadIdx.x] = g_b3[threadIdx.x];
  __syncthreads();

  const long long total = min(crd.total_ptr ? (long long)*crd.total_ptr : crd.total_direct, crd.capacity);
  const int A = d.app_dim, F = d.fea_pe, V = d.view_pe;
  const int base_s = A + 3, base_c = base_s + A * F, base_vs = base_c + A * F, base_vc = base_vs + 3 * V;

  for (long long tile = (long long)blockIdx.x * TM; tile < total; tile += (long long)gridDim.x * TM) {
    // ---- build the input tile: 4 threads per sample -------------------------------------
    {
      const int m = threadIdx.x & (TM - 1), q = threadIdx.x >> 6;
      const long long j = tile + m;
      const bool live = j < total;
      const float* fr = feat + (size_t)(live ? j : 0) * d.feat_stride;
      float view[3] = {0.0f, 0.0f, 0.0f};
      if (live) {
        const float* vsrc;
        if (crd.view_direct) {
          vsrc = crd.view_direct + (size_t)j * crd.point_stride;
        } else {
          const uint32_t ray = __ldg(crd.ids + (crd.index ? (long long)__ldg(crd.index + j) : j)) >> kbits;
          vsrc = crd.rays + (size_t)ray * 6 + 3;
        }
        view[0] = __ldg(vsrc + 0);
        view[1] = __ldg(vsrc + 1);
        view[2] = __ldg(vsrc + 2);
      }
      for (int it = q; it < A + 3; it += 4) xa[it * TM + m] = live ? (it < A ? __ldg(fr + it) : view[it - A]) : 0.0f;
      for (int idx = q; idx < A * F; idx += 4) {
        const int i = idx / F, f = idx - i * F;
        float s = 0.0f, c = 0.0f;
        if (live) sincosf(__ldg(fr + i) * (float)(1 << f), &s, &c);
        xa[(base_s + idx) * TM + m] = s;
        xa[(base_c + idx) * TM + m] = c;
      }
      for (int idx = q; idx < 3 * V; idx += 4) {
        const int i = idx / V, f = idx - i * V;
        float s = 0.0f, c = 0.0f;
        if (live) sincosf(view[i] * (float)(1 << f), &s, &c);
        xa[(base_vs + idx) * TM + m] = s;
        xa[(base_vc + idx) * TM + m] = c;
      }
      for (int it = d.in_dim + q; it < d.k1_pad; it += 4) xa[it * TM + m] = 0.0f;
    }
    __syncthreads();
    dense_relu<0>(w1t, b1, xa, xb, d.k1_pad);
    __syncthreads();
    dense_relu<1>(w2t, b2, xb, xa, HID);
    __syncthreads();
    if (threadIdx.x < 3 * TM) {
      const int c = threadIdx.x / TM, m = threadIdx.x - c * TM;
      float acc = 0.0f;
#pragma unroll 8
      for (int n = 0; n < HID; ++n) acc = fmaf(w3[c * HID + n], xa[n * TM + m], acc);
      acc += b3[c];
      const long long j = tile + m;
      if (j < total) rgb_out[(size_t)j * 3 + c] = 1.0f / (1.0f + expf(-acc));
    }
    __syncthreads();
  }
}

}  // namespace

int launch_mlp_simt(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, int feat_stride, const float* feat,
                    float* rgb, cudaStream_t st) {
  if (m->cfg.hidden != HID) {
    gnr_set_error("fp32 MLP kernel supports featureC == %d (got %d)", HID, m->cfg.hidden);
    return -1;
  }
  MlpDims d;
  d.app_dim = m->cfg.app_dim;
  d.fea_pe = m->cfg.fea_pe;
  d.view_pe = m->cfg.view_pe > 0 ? m->cfg.view_pe : 0;
  d.in_dim = m->mlp.in_dim;
  d.k1_pad = m->mlp.k1_pad;
  d.feat_stride = feat_stride;
  size_t smem = ((size_t)d.k1_pad * HID + HID * HID + 3 * HID + 2 * HID + 4 + (size_t)d.k1_pad * TM + HID * TM) * sizeof(float);
  if (smem > 227 * 1024) {
    gnr_set_error("fp32 MLP kernel: input width %d needs %zu bytes of shared memory", d.in_dim, smem);
    return -1;
  }
  cudaFuncSetAttribute(mlp_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  mlp_simt_kernel<<<m->sm_count, kThreads, smem, st>>>(d, p.kbits, c, feat, m->mlp.w1t, m->mlp.w2t, m->mlp.w3, m->mlp.b1,
                                                       m->mlp.b2, m->mlp.b3, rgb);
  return (int)cudaGetLastError();
}
