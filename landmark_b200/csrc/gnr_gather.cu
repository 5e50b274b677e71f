// VM feature gather: bilinear plane x linear line, channel-last planes.
//
// Two families of kernels.  The general ones (density_kernel, app_gather_kernel,
// app_products_kernel; any channel count, list or point mode) let four lanes share one sample:
// lane c4 owns channels {16 j + 4 c4 .. +3 : j < J}, so one 128-bit load instruction of a warp reads
// 8 samples x 64 contiguous bytes.  The ones the frame loop runs (march_kernel,
// app_products_thread_kernel) give a whole sample to one thread and neighbouring rays to the lanes
// of a warp, with 256-bit loads; per sample they perform the same operations in the same order as
// the four-lane kernels, so both families give the same bits (except the appearance gather from
// fp16 planes, which interpolates in packed fp16).  Interpolation follows
// F.grid_sample(mode="bilinear", padding_mode="zeros", align_corners=True) as called by
// compute_densityfeature / compute_appfeature (app/models/gridnerf_sequential.py:779-871):
// index = ((x + 1) / 2) * (size - 1); the weight of a corner is the product of the distances
// to the opposite corner; taps outside the grid contribute zero.
#include <cuda_fp16.h>

#include "gnr_gather.cuh"

namespace {

constexpr int kBlock = 256;
constexpr int kFeat = 28;  // accumulators per sample for the basis projection (app_dim <= 28)


// float4 arithmetic as two packed fp32x2 instructions each (sm_100 has paired FP32 pipes)
__device__ __forceinline__ float4 f4_scale(float4 a, float s) {
  const float2 ss = make_float2(s, s);
  const float2 lo = __fmul2_rn(make_float2(a.x, a.y), ss), hi = __fmul2_rn(make_float2(a.z, a.w), ss);
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ float4 f4_fma(float4 a, float s, float4 c) {
  const float2 ss = make_float2(s, s);
  const float2 lo = __ffma2_rn(make_float2(a.x, a.y), ss, make_float2(c.x, c.y));
  const float2 hi = __ffma2_rn(make_float2(a.z, a.w), ss, make_float2(c.z, c.w));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ float4 f4_mul(float4 a, float4 b) {
  const float2 lo = __fmul2_rn(make_float2(a.x, a.y), make_float2(b.x, b.y));
  const float2 hi = __fmul2_rn(make_float2(a.z, a.w), make_float2(b.z, b.w));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// Products plane(x, y) * line(l) for the 4 J channels this lane owns.
// Valid samples lie inside the closed box, so the continuous index is clamped to the grid
// and the lower corner to size - 2: no tap can fall outside and no bounds test is needed (a
// point exactly on the upper face then takes the last texel with weight 1, which is what
// zero padding gives as well).  All offsets are 32-bit float4 indices.
// The four channels 16 j + 4 c4 .. + 3 of texel `texel` (C channels per texel) from an fp32 or an
// fp16 array.
template <bool HALF>
__device__ __forceinline__ float4 load4(const float* base, uint32_t texel, uint32_t C, int c4, int j) {
  if constexpr (HALF) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(base) + ((texel * C) >> 2) + c4 + 4 * j);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
  } else {
    return __ldg(reinterpret_cast<const float4*>(base) + ((texel * C) >> 2) + c4 + 4 * j);
  }
}

template <int J, bool HALF = false>
__device__ __forceinline__ void pair_products_tap(const GnrPlane& pl, Tap tx, Tap ty, Tap tl, int c4, float4 (&prod)[J]) {
  const float ax1 = tx.f1, ay1 = ty.f1, al1 = tl.f1;
  const float ax0 = 1.0f - ax1, ay0 = 1.0f - ay1, al0 = 1.0f - al1;
  const float w_nw = ax0 * ay0, w_ne = ax1 * ay0, w_sw = ax0 * ay1, w_se = ax1 * ay1;
  const uint32_t C = (uint32_t)pl.C;
  const uint32_t nw = (uint32_t)ty.i0 * (uint32_t)pl.W + (uint32_t)tx.i0, sw = nw + (uint32_t)pl.W;
  const uint32_t ln = (uint32_t)tl.i0;
  float4 v_nw[J], v_ne[J], v_sw[J], v_se[J], v_l0[J], v_l1[J];
#pragma unroll
  for (int j = 0; j < J; ++j) {
    v_nw[j] = load4<HALF>(pl.plane, nw, C, c4, j);
    v_ne[j] = load4<HALF>(pl.plane, nw + 1u, C, c4, j);
    v_sw[j] = load4<HALF>(pl.plane, sw, C, c4, j);
    v_se[j] = load4<HALF>(pl.plane, sw + 1u, C, c4, j);
    v_l0[j] = load4<HALF>(pl.line, ln, C, c4, j);
    v_l1[j] = load4<HALF>(pl.line, ln + 1u, C, c4, j);
  }
#pragma unroll
  for (int j = 0; j < J; ++j) {
    float4 pv = f4_scale(v_nw[j], w_nw);
    pv = f4_fma(v_ne[j], w_ne, pv);
    pv = f4_fma(v_sw[j], w_sw, pv);
    pv = f4_fma(v_se[j], w_se, pv);
    float4 lv = f4_fma(v_l1[j], al1, f4_scale(v_l0[j], al0));
    prod[j] = f4_mul(pv, lv);
  }
}

template <int J>
__device__ __forceinline__ void pair_products(const GnrPlane& pl, float x, float y, float z, int c4, float4 (&prod)[J]) {
  const float u = pick(x, y, z, pl.mat0), v = pick(x, y, z, pl.mat1), l = pick(x, y, z, pl.vec);
  pair_products_tap<J>(pl, make_tap(u, pl.fw, pl.W), make_tap(v, pl.fh, pl.H), make_tap(l, pl.fl, pl.L), c4, prod);
}

// The three plane/line pairs of one sample.  NP == 3 is the standard VM layout (pairs
// (x,y|z), (x,z|y), (y,z|x) on one grid, verified by the host): its nine coordinate lookups
// collapse into three.  NP == 0 walks planes.n pairs generically.
template <int J, int NP, bool HALF = false, class F>
__device__ __forceinline__ void for_each_pair(const PlaneSet& planes, float x, float y, float z, int c4, F&& f) {
  auto one = [&](const GnrPlane& pl, Tap ta, Tap tb, Tap tl, float4(&prod)[J]) {
    pair_products_tap<J, HALF>(pl, ta, tb, tl, c4, prod);
  };
  if (NP == 3) {
    const Tap tx = make_tap(x, planes.p[0].fw, planes.p[0].W);
    const Tap ty = make_tap(y, planes.p[0].fh, planes.p[0].H);
    const Tap tz = make_tap(z, planes.p[0].fl, planes.p[0].L);
    float4 prod[J];
    one(planes.p[0], tx, ty, tz, prod);
    f(0, prod);
    one(planes.p[1], tx, tz, ty, prod);
    f(1, prod);
    one(planes.p[2], ty, tz, tx, prod);
    f(2, prod);
  } else {
    for (int pi = 0; pi < planes.n; ++pi) {
      const GnrPlane& pl = planes.p[pi];
      const float u = pick(x, y, z, pl.mat0), v = pick(x, y, z, pl.mat1), l = pick(x, y, z, pl.vec);
      float4 prod[J];
      one(pl, make_tap(u, pl.fw, pl.W), make_tap(v, pl.fh, pl.H), make_tap(l, pl.fl, pl.L), prod);
      f(pi, prod);
    }
  }
}

// ---- one thread, one sample: all channels of a pair with 256-bit loads ----------------------------
struct __align__(32) F8 {
  float4 lo, hi;
};
__device__ __forceinline__ F8 ldg8(const float* ptr) {
  F8 r;
  asm("ld.global.nc.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=f"(r.lo.x), "=f"(r.lo.y), "=f"(r.lo.z), "=f"(r.lo.w), "=f"(r.hi.x), "=f"(r.hi.y), "=f"(r.hi.z), "=f"(r.hi.w)
      : "l"(ptr));
  return r;
}

// Adds to part[c] (c = 0..3) the sum over j of the plane x line products of channels
// 16 j + 4 c .. 16 j + 4 c + 3, with the operations and the order the four lanes of a quad use in
// pair_products_tap / density_kernel, so that a sample's density feature has the same bits
// whichever kernel computes it.
// Eight consecutive channels starting at channel 8 h of a texel, fp32 (one 256-bit load) or fp16 (one
// 128-bit load).
template <bool HALF>
__device__ __forceinline__ F8 load8c(const float* base, uint32_t texel, uint32_t C, int h) {
  if constexpr (HALF) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(base) + ((texel * C) >> 3) + h);
    const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&a.x)), a1 = __half22float2(*reinterpret_cast<const __half2*>(&a.y));
    const float2 a2 = __half22float2(*reinterpret_cast<const __half2*>(&a.z)), a3 = __half22float2(*reinterpret_cast<const __half2*>(&a.w));
    F8 r;
    r.lo = make_float4(a0.x, a0.y, a1.x, a1.y);
    r.hi = make_float4(a2.x, a2.y, a3.x, a3.y);
    return r;
  } else {
    return ldg8(base + (size_t)texel * C + 8 * h);
  }
}

template <int J, bool HALF = false>
__device__ __forceinline__ void pair_sums_thread(const GnrPlane& pl, Tap tx, Tap ty, Tap tl, float (&part)[4]) {
  const float ax1 = tx.f1, ay1 = ty.f1, al1 = tl.f1;
  const float ax0 = 1.0f - ax1, ay0 = 1.0f - ay1, al0 = 1.0f - al1;
  const float w_nw = ax0 * ay0, w_ne = ax1 * ay0, w_sw = ax0 * ay1, w_se = ax1 * ay1;
  constexpr uint32_t C = 16u * J;
  const uint32_t nw_t = (uint32_t)ty.i0 * (uint32_t)pl.W + (uint32_t)tx.i0, sw_t = nw_t + (uint32_t)pl.W;
  const uint32_t l_t = (uint32_t)tl.i0;
  float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int h = 0; h < 2 * J; ++h) {  // 8 channels per round: quarters 2 (h & 1) and 2 (h & 1) + 1 of group j = h >> 1
    const F8 v_nw = load8c<HALF>(pl.plane, nw_t, C, h), v_ne = load8c<HALF>(pl.plane, nw_t + 1u, C, h);
    const F8 v_sw = load8c<HALF>(pl.plane, sw_t, C, h), v_se = load8c<HALF>(pl.plane, sw_t + 1u, C, h);
    const F8 v_l0 = load8c<HALF>(pl.line, l_t, C, h), v_l1 = load8c<HALF>(pl.line, l_t + 1u, C, h);
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const float4 nw = q ? v_nw.hi : v_nw.lo, ne = q ? v_ne.hi : v_ne.lo, sw = q ? v_sw.hi : v_sw.lo, se = q ? v_se.hi : v_se.lo;
      const float4 l0 = q ? v_l0.hi : v_l0.lo, l1 = q ? v_l1.hi : v_l1.lo;
      float4 pv = f4_scale(nw, w_nw);
      pv = f4_fma(ne, w_ne, pv);
      pv = f4_fma(sw, w_sw, pv);
      pv = f4_fma(se, w_se, pv);
      const float4 lv = f4_fma(l1, al1, f4_scale(l0, al0));
      const float4 prod = f4_mul(pv, lv);
      s[2 * (h & 1) + q] += (prod.x + prod.y) + (prod.z + prod.w);
    }
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) part[c] += s[c];
}

// Density feature of one sample, computed by one thread.
template <int J, int NP, bool HALF = false>
__device__ __forceinline__ float density_thread(const PlaneSet& planes, float x, float y, float z) {
  float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (NP == 3) {
    const Tap tx = make_tap(x, planes.p[0].fw, planes.p[0].W);
    const Tap ty = make_tap(y, planes.p[0].fh, planes.p[0].H);
    const Tap tz = make_tap(z, planes.p[0].fl, planes.p[0].L);
    pair_sums_thread<J, HALF>(planes.p[0], tx, ty, tz, part);
    pair_sums_thread<J, HALF>(planes.p[1], tx, tz, ty, part);
    pair_sums_thread<J, HALF>(planes.p[2], ty, tz, tx, part);
  } else {
    for (int pi = 0; pi < planes.n; ++pi) {
      const GnrPlane& pl = planes.p[pi];
      const float u = pick(x, y, z, pl.mat0), v = pick(x, y, z, pl.mat1), l = pick(x, y, z, pl.vec);
      pair_sums_thread<J, HALF>(pl, make_tap(u, pl.fw, pl.W), make_tap(v, pl.fh, pl.H), make_tap(l, pl.fl, pl.L), part);
    }
  }
  return (part[0] + part[1]) + (part[2] + part[3]);
}

// ---- density from the pre-summed lattice ---------------------------------------------------------
// For the standard three-pair layout on one grid the density feature
//   sum_pairs sum_c bilinear(plane_c)(a, b) * linear(line_c)(l)
// is, term by term, the trilinear interpolation of the products plane_c[j][i] * line_c[k], hence
// of their sum over channels and pairs: one scalar per lattice point,
//   V[x][y][z] = sum_c P0_c[y][x] L0_c[z] + P1_c[z][x] L1_c[y] + P2_c[z][y] L2_c[x],
// interpolated with the same lower indices and fractions (make_tap) the plane/line taps use.  The
// function is the same; only the order of the floating-point sums differs (a few 1e-8 on the
// feature).  A sample then costs 8 scalar loads instead of 36 loads of 32 bytes.
// z is the fastest axis of V: a ray's consecutive samples and the two z taps share sectors.
__device__ __forceinline__ float lattice_feature(const float* __restrict__ V, uint32_t Gy, uint32_t Gz, Tap tx, Tap ty, Tap tz) {
  const uint32_t b00 = ((uint32_t)tx.i0 * Gy + (uint32_t)ty.i0) * Gz + (uint32_t)tz.i0;
  const uint32_t b01 = b00 + Gz, b10 = b00 + Gy * Gz, b11 = b10 + Gz;
  const float v000 = __ldg(V + b00), v001 = __ldg(V + b00 + 1u), v010 = __ldg(V + b01), v011 = __ldg(V + b01 + 1u);
  const float v100 = __ldg(V + b10), v101 = __ldg(V + b10 + 1u), v110 = __ldg(V + b11), v111 = __ldg(V + b11 + 1u);
  const float fz = tz.f1, fy = ty.f1, fx = tx.f1;
  const float c00 = fmaf(fz, v001 - v000, v000), c01 = fmaf(fz, v011 - v010, v010);
  const float c10 = fmaf(fz, v101 - v100, v100), c11 = fmaf(fz, v111 - v110, v110);
  const float c0 = fmaf(fy, c01 - c00, c00), c1 = fmaf(fy, c11 - c10, c10);
  return fmaf(fx, c1 - c0, c0);
}

struct LatticeRef {
  const float* v;  // null: gather from the planes and lines
  int gx, gy, gz;
};

__device__ __forceinline__ float lattice_density_feature(const LatticeRef& lat, const PlaneSet& planes, float x, float y, float z) {
  const Tap tx = make_tap(x, planes.p[0].fw, planes.p[0].W);
  const Tap ty = make_tap(y, planes.p[0].fh, planes.p[0].H);
  const Tap tz = make_tap(z, planes.p[0].fl, planes.p[0].L);
  return lattice_feature(lat.v, (uint32_t)lat.gy, (uint32_t)lat.gz, tx, ty, tz);
}

// One thread per lattice point, z fastest.  The 48 (3 x C) products are summed in double and
// rounded once, so every lattice value is the correctly rounded sum.
template <bool HALF>
__global__ void __launch_bounds__(256)
build_lattice_kernel(PlaneSet planes, int C, int gx, int gy, int gz, float* __restrict__ V) {
  const long long total = (long long)gx * gy * gz;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int z = (int)(i % gz), y = (int)((i / gz) % gy), x = (int)(i / ((long long)gz * gy));
    // texel (plane) and entry (line) of every pair for this lattice point
    const size_t pt[3] = {(size_t)y * planes.p[0].W + x, (size_t)z * planes.p[1].W + x, (size_t)z * planes.p[2].W + y};
    const size_t ln[3] = {(size_t)z, (size_t)y, (size_t)x};
    double acc = 0.0;
#pragma unroll
    for (int pi = 0; pi < 3; ++pi) {
      for (int c = 0; c < C; ++c) {
        float pv, lv;
        if constexpr (HALF) {
          pv = __half2float(reinterpret_cast<const __half*>(planes.p[pi].plane)[pt[pi] * C + c]);
          lv = __half2float(reinterpret_cast<const __half*>(planes.p[pi].line)[ln[pi] * C + c]);
        } else {
          pv = __ldg(planes.p[pi].plane + pt[pi] * C + c);
          lv = __ldg(planes.p[pi].line + ln[pi] * C + c);
        }
        acc += (double)pv * (double)lv;
      }
    }
    V[i] = (float)acc;
  }
}

__device__ __forceinline__ float density_activation(float f, float shift, int act) {
  if (act == 1) return fmaxf(f, 0.0f);
  // F.softplus (beta 1, threshold 20): log1p(exp(x)).  exp by the hardware approximation; log1p
  // by its series while exp(x) is small (where 1 + e would round e away) and by log(1 + e) above.
  const float x = f + shift;
  if (x > 20.0f) return x;
  const float e = __expf(x);
  return e < 0.01f ? e * (1.0f - e * (0.5f - e * 0.33333334f)) : __logf(1.0f + e);
}

// Contiguous share of [0, total) for this CTA, in units of the kBlock / LANES samples one CTA
// iteration covers (LANES lanes share a sample).
template <int LANES = 4>
__device__ __forceinline__ void cta_range(long long total, long long& beg, long long& end) {
  constexpr long long kStep = kBlock / LANES;
  const long long steps = (total + kStep - 1) / kStep;
  const long long per = (steps + gridDim.x - 1) / gridDim.x;
  beg = min(total, (long long)blockIdx.x * per * kStep);
  end = min(total, beg + per * kStep);
}

template <int J, int NP, bool HALF = false>
__global__ void __launch_bounds__(kBlock)
density_kernel(GnrSampleParams p, PlaneSet planes, GnrCoords crd, float shift, int act, float* __restrict__ sigma_feat,
               float* __restrict__ sigma) {
  const int c4 = threadIdx.x & 3;
  const long long total = coords_total(crd);
  // Each CTA walks one contiguous range of the (ray-major) list, so that the texels a ray
  // touches are still in this SM's L1 when the next samples and the neighbouring ray need them.
  long long range_beg, range_end;
  cta_range(total, range_beg, range_end);
  // whole warps iterate together so that the quad shuffles below are always convergent
  for (long long base = range_beg + (threadIdx.x >> 5) * 8; base < range_end; base += kBlock / 4) {
    const long long i = base + ((threadIdx.x & 31) >> 2);
    const bool active = i < range_end;
    float acc = 0.0f;
    if (active) {
      float x, y, z;
      sample_xyz(p, crd, i, x, y, z);
      for_each_pair<J, NP, HALF>(planes, x, y, z, c4, [&](int, const float4(&prod)[J]) {
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < J; ++j) s += (prod[j].x + prod[j].y) + (prod[j].z + prod[j].w);
        acc += s;
      });
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    if (active && c4 == 0) {
      if (sigma_feat) sigma_feat[i] = acc;
      sigma[i] = density_activation(acc, shift, act);
    }
  }
}

// Appearance lattice: the 27 projected features at every grid point,
//   A_o[x][y][z] = sum over pairs p and channels c of basis[o][p][c] * plane_p,c(texel) * line_p,c(entry),
// stored as 32 fp16 channels per point in the order the one-kernel appearance path reads them: channels
// 0..13 = features 0..13, 14..15 = 0, 16..28 = features 14..26, 29..31 = 0 (each of the two threads of a
// row loads its own 32 bytes per tap).  One thread per grid point; the basis matrix sits in shared memory
// as [pair * 48 + c][28] so that a warp reads it as broadcasts; sums in fp32, one rounding to fp16.
template <bool HALF>
__global__ void __launch_bounds__(128)
build_app_lattice_kernel(PlaneSet planes, const float* __restrict__ basis, int app_dim, int n_app, int gx, int gy, int gz,
                         __half* __restrict__ V) {
  extern __shared__ float s_basis[];  // [3 * 48][28]
  for (int i = threadIdx.x; i < 3 * 48 * 28; i += blockDim.x) {
    const int k = i / 28, o = i - k * 28, pi = k / 48, c = k - pi * 48;
    s_basis[i] = (o < app_dim && c < n_app) ? basis[(size_t)o * (3 * n_app) + pi * n_app + c] : 0.0f;
  }
  __syncthreads();
  const long long total = (long long)gx * gy * gz;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int z = (int)(i % gz), y = (int)((i / gz) % gy), x = (int)(i / ((long long)gz * gy));
    const size_t pt[3] = {(size_t)y * planes.p[0].W + x, (size_t)z * planes.p[1].W + x, (size_t)z * planes.p[2].W + y};
    const size_t ln[3] = {(size_t)z, (size_t)y, (size_t)x};
    float acc[28];
#pragma unroll
    for (int o = 0; o < 28; ++o) acc[o] = 0.0f;
#pragma unroll 1
    for (int pi = 0; pi < 3; ++pi) {
#pragma unroll 4
      for (int c = 0; c < 48; ++c) {
        float pv, lv;
        if constexpr (HALF) {
          pv = __half2float(reinterpret_cast<const __half*>(planes.p[pi].plane)[pt[pi] * 48 + c]);
          lv = __half2float(reinterpret_cast<const __half*>(planes.p[pi].line)[ln[pi] * 48 + c]);
        } else {
          pv = __ldg(planes.p[pi].plane + pt[pi] * 48 + c);
          lv = __ldg(planes.p[pi].line + ln[pi] * 48 + c);
        }
        const float prod = pv * lv;
        const float4* w = reinterpret_cast<const float4*>(s_basis + (pi * 48 + c) * 28);
#pragma unroll
        for (int q = 0; q < 7; ++q) {
          const float4 wq = w[q];
          acc[4 * q + 0] = fmaf(prod, wq.x, acc[4 * q + 0]);
          acc[4 * q + 1] = fmaf(prod, wq.y, acc[4 * q + 1]);
          acc[4 * q + 2] = fmaf(prod, wq.z, acc[4 * q + 2]);
          acc[4 * q + 3] = fmaf(prod, wq.w, acc[4 * q + 3]);
        }
      }
    }
    __half out[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) out[e] = __float2half_rn(0.0f);
#pragma unroll
    for (int o = 0; o < 14; ++o) out[o] = __float2half_rn(acc[o]);
#pragma unroll
    for (int o = 14; o < 27; ++o) out[16 + (o - 14)] = __float2half_rn(acc[o]);
    uint4* dst = reinterpret_cast<uint4*>(V + (size_t)i * 32);
    const uint4* src = reinterpret_cast<const uint4*>(out);
#pragma unroll
    for (int q = 0; q < 4; ++q) dst[q] = src[q];
  }
}

// List / point mode density from the lattice: one thread per item.
__global__ void __launch_bounds__(kBlock)
density_lattice_kernel(GnrSampleParams p, PlaneSet planes, LatticeRef lat, GnrCoords crd, float shift, int act,
                       float* __restrict__ sigma_feat, float* __restrict__ sigma) {
  const long long total = coords_total(crd);
  for (long long i = (long long)blockIdx.x * kBlock + threadIdx.x; i < total; i += (long long)gridDim.x * kBlock) {
    float x, y, z;
    sample_xyz(p, crd, i, x, y, z);
    const float f = lattice_density_feature(lat, planes, x, y, z);
    if (sigma_feat) sigma_feat[i] = f;
    sigma[i] = density_activation(f, shift, act);
  }
}

// Fused density + weights pass ("march"): one thread walks one ray's valid samples (the set bits of
// its validity words; sample j of the ray owns entry offsets[ray] + j of the per-sample arrays): density feature (density_thread), activation, raw2alpha's alpha, the
// running transmittance product in sample order (as torch.cumprod computes it on the CPU), weight,
// and the ray's accumulated opacity and depth.  The 32 rays of a warp are consecutive rays of the
// chunk; when those are neighbouring pixels (tile order) their samples of equal rank lie within a
// few voxels of each other, so the lanes of one load instruction read a handful of texels and the
// L1 serves them as broadcasts.  When the transmittance falls below t_stop the ray stops: the
// remaining samples get weight 0 and never touch the planes.  What they would have added to acc
// (and, with a white background, taken from rgb) is bounded by the transmittance at the stop,
// i.e. by t_stop.  With t_stop == 0 the weights are bit-identical to density_kernel followed by
// weights_kernel.
constexpr int kMarchBlock = 32;  // one warp per CTA: a finished warp frees its slot at once

template <int J, int NP, bool HALF = false, bool LAT = false>
__global__ void __launch_bounds__(kMarchBlock, LAT ? 32 : 16)
march_kernel(GnrSampleParams p, PlaneSet planes, LatticeRef lat, const float* __restrict__ rays, const float* __restrict__ t_min_arr,
             const uint32_t* __restrict__ words, const int32_t* __restrict__ offsets, long long n_rays, long long capacity,
             float shift, int act, float distance_scale, float thres, float t_stop, float* __restrict__ weight,
             float* __restrict__ acc_out, float* __restrict__ depth_out, int32_t* __restrict__ app_counts,
             int32_t* __restrict__ evaluated_total, int list_only, float2* __restrict__ packed) {
  __shared__ int s_evaluated;
  if (threadIdx.x == 0) s_evaluated = 0;
  __syncthreads();
  const long long ray = (long long)blockIdx.x * kMarchBlock + threadIdx.x;
  int evaluated = 0;
  if (ray < n_rays) {
    const long long beg = offsets[ray], end = min((long long)offsets[ray + 1], capacity);
    float acc = 0.0f, dep = 0.0f;
    int n_app = 0;
    if (beg < end) {
      const float* r = rays + (size_t)ray * 6;
      const float ox = __ldg(r + 0), oy = __ldg(r + 1), oz = __ldg(r + 2);
      const float dx = __ldg(r + 3), dy = __ldg(r + 4), dz = __ldg(r + 5);
      const float t_min = t_min_arr[ray];
      float T = 1.0f;
      long long i = beg;
      // the ray's valid samples are the set bits of its validity words, in order
      const uint32_t* wrow = words + (size_t)ray * p.words;
      int word = 0;
      uint32_t bits = __ldg(wrow);
      while (i < end) {
        while (bits == 0u && word + 1 < p.words) bits = __ldg(wrow + ++word);
        if (bits == 0u) break;  // (cannot happen: offsets count exactly the set bits)
        const int k = word * 32 + (__ffs(bits) - 1);
        bits &= bits - 1u;
        const float t = gnr_sample_t(p, t_min, k);
        const float x = gnr_normalize(gnr_point(ox, dx, t), p.lo[0], p.inv[0]);
        const float y = gnr_normalize(gnr_point(oy, dy, t), p.lo[1], p.inv[1]);
        const float z = gnr_normalize(gnr_point(oz, dz, t), p.lo[2], p.inv[2]);
        float feat;
        if constexpr (LAT) feat = lattice_density_feature(lat, planes, x, y, z);
        else feat = density_thread<J, NP, HALF>(planes, x, y, z);
        const float sg = density_activation(feat, shift, act);
        const float dist = (k == p.S - 1) ? 0.0f : __fsub_rn(gnr_sample_t(p, t_min, k + 1), t);
        const float alpha = __fsub_rn(1.0f, expf(__fmul_rn(-sg, __fmul_rn(dist, distance_scale))));
        const float w = alpha * T;
        if (list_only) {
          // the frame loop reads nothing but the samples that pass the appearance threshold: they go, as (weight,
          // sample number) pairs of 8 bytes, to the front of the ray's own range of the pair array, in order
          if (w > thres) packed[beg + n_app] = make_float2(w, __int_as_float(k));
        } else {
          weight[i] = w;
        }
        acc += w;
        dep = fmaf(w, t, dep);
        n_app += (w > thres) ? 1 : 0;
        T *= __fadd_rn(__fsub_rn(1.0f, alpha), 1e-10f);
        ++i;
        if (T < t_stop) break;
      }
      evaluated = (int)(i - beg);
      // Weights behind the stop are zero (written for callers that look at the weight array itself).
      if (!list_only)
        for (; i < end; ++i) weight[i] = 0.0f;
    }
    acc_out[ray] = acc;
    depth_out[ray] = dep;
    app_counts[ray] = n_app;
  }
  evaluated = __reduce_add_sync(0xffffffffu, evaluated);
  if ((threadIdx.x & 31) == 0 && evaluated) atomicAdd(&s_evaluated, evaluated);
  __syncthreads();
  if (threadIdx.x == 0 && s_evaluated) atomicAdd(evaluated_total, s_evaluated);
}

// Appearance gather + basis projection.  The basis weights sit in shared memory, blocked per
// (pair, lane-in-quad): row t = 4 j + e of block (pair, c4) holds the `app_dim` weights of
// channel 16 j + 4 c4 + e of that pair, padded to kFeat floats; blocks are padded by 8 floats
// so that the four lanes of a quad read disjoint banks.
template <int J>
__global__ void __launch_bounds__(kBlock)
app_gather_kernel(GnrSampleParams p, PlaneSet planes, GnrCoords crd, const float* __restrict__ basis_blocked,
                  int feat_stride, float* __restrict__ feat_out) {
  extern __shared__ float4 smem_f4[];
  float* wsm = reinterpret_cast<float*>(smem_f4);
  constexpr int kBlk = 4 * J * kFeat + 8;
  const int n_w = planes.n * 4 * kBlk;
  for (int i = threadIdx.x; i < n_w; i += kBlock) wsm[i] = basis_blocked[i];
  __syncthreads();

  const int c4 = threadIdx.x & 3;
  const long long total = coords_total(crd);
  long long range_beg, range_end;
  cta_range(total, range_beg, range_end);
  for (long long base = range_beg + (threadIdx.x >> 5) * 8; base < range_end; base += kBlock / 4) {
    const long long j_app = base + ((threadIdx.x & 31) >> 2);
    const bool active = j_app < range_end;
    float acc[kFeat];
#pragma unroll
    for (int o = 0; o < kFeat; ++o) acc[o] = 0.0f;
    if (active) {
      float x, y, z;
      sample_xyz(p, crd, j_app, x, y, z);
      for (int pi = 0; pi < planes.n; ++pi) {
        float4 prod[J];
        pair_products<J>(planes.p[pi], x, y, z, c4, prod);
        const float* wb = wsm + (pi * 4 + c4) * kBlk;
#pragma unroll
        for (int j = 0; j < J; ++j) {
          const float pv[4] = {prod[j].x, prod[j].y, prod[j].z, prod[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float4* wrow = reinterpret_cast<const float4*>(wb + (j * 4 + e) * kFeat);
#pragma unroll
            for (int q = 0; q < kFeat / 4; ++q) {
              const float4 w = wrow[q];
              acc[4 * q + 0] = fmaf(pv[e], w.x, acc[4 * q + 0]);
              acc[4 * q + 1] = fmaf(pv[e], w.y, acc[4 * q + 1]);
              acc[4 * q + 2] = fmaf(pv[e], w.z, acc[4 * q + 2]);
              acc[4 * q + 3] = fmaf(pv[e], w.w, acc[4 * q + 3]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int o = 0; o < kFeat; ++o) {
      acc[o] += __shfl_xor_sync(0xffffffffu, acc[o], 1);
      acc[o] += __shfl_xor_sync(0xffffffffu, acc[o], 2);
    }
    if (active && c4 == 0) {
      float4* out = reinterpret_cast<float4*>(feat_out + (size_t)j_app * feat_stride);
#pragma unroll
      for (int q = 0; q < kFeat / 4; ++q)
        if (4 * q < feat_stride) out[q] = make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
    }
  }
}

// Appearance gather for the tensor-core path: the plane x line products themselves are the
// K dimension of the basis projection, so they are written as fp16 straight into the MMA
// operand layout of their 128-sample tile: element (row r, k) of tile t at byte
//   t * tile_bytes + (k / 8) * 2048 + r * 16 + (k % 8) * 2,     k = pair * C + channel.
// With TA == 2 the fp16 rounding residual goes to a second image of the same shape.
// One more 16-byte group per row, after the products (k group `view_group`), carries the
// sample's view direction for the MLP kernel as fp16 pairs {hi x, hi y, hi z, lo x, lo y, lo z}:
// hi + lo restores the fp32 value to about 2^-22, and the MLP kernel needs no list lookups.
// (fp32 planes only; fp16 storage goes through app_products_thread_kernel.)
template <int J, int NP, int TA>
__global__ void __launch_bounds__(kBlock)
app_products_kernel(GnrSampleParams p, PlaneSet planes, GnrCoords crd, unsigned char* __restrict__ prod_hi,
                    unsigned char* __restrict__ prod_lo, int tile_bytes, int view_group) {
  const int c4 = threadIdx.x & 3;
  const long long total = coords_total(crd);
  long long range_beg, range_end;
  cta_range(total, range_beg, range_end);
  for (long long base = range_beg + (threadIdx.x >> 5) * 8; base < range_end; base += kBlock / 4) {
    const long long j_app = base + ((threadIdx.x & 31) >> 2);
    if (j_app >= range_end) continue;
    float x, y, z, view[3];
    sample_xyz(p, crd, j_app, x, y, z, view);
    const long long tile = j_app >> 7;
    const int row = (int)(j_app & 127);
    const size_t out0 = (size_t)tile * tile_bytes + (size_t)row * 16 + (size_t)(c4 & 1) * 8;
    if (c4 == 0) {
      const __half hx = __float2half_rn(view[0]), hy = __float2half_rn(view[1]), hz = __float2half_rn(view[2]);
      const __half2 a = __halves2half2(hx, hy);
      const __half2 b = __halves2half2(hz, __float2half_rn(view[0] - __half2float(hx)));
      const __half2 c = __floats2half2_rn(view[1] - __half2float(hy), view[2] - __half2float(hz));
      uint4 vv;
      vv.x = *reinterpret_cast<const uint32_t*>(&a);
      vv.y = *reinterpret_cast<const uint32_t*>(&b);
      vv.z = *reinterpret_cast<const uint32_t*>(&c);
      vv.w = 0u;
      *reinterpret_cast<uint4*>(prod_hi + (size_t)tile * tile_bytes + (size_t)view_group * 2048 + (size_t)row * 16) = vv;
    }
    for_each_pair<J, NP>(planes, x, y, z, c4, [&](int pi, const float4(&prod)[J]) {
#pragma unroll
      for (int j = 0; j < J; ++j) {
        const size_t at = out0 + (size_t)(pi * 2 * J + 2 * j + (c4 >> 1)) * 2048;
        const __half2 h0 = __floats2half2_rn(prod[j].x, prod[j].y), h1 = __floats2half2_rn(prod[j].z, prod[j].w);
        uint2 hv;
        hv.x = *reinterpret_cast<const uint32_t*>(&h0);
        hv.y = *reinterpret_cast<const uint32_t*>(&h1);
        *reinterpret_cast<uint2*>(prod_hi + at) = hv;
        if (TA == 2) {
          const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
          const __half2 l0 = __floats2half2_rn(prod[j].x - f0.x, prod[j].y - f0.y);
          const __half2 l1 = __floats2half2_rn(prod[j].z - f1.x, prod[j].w - f1.y);
          uint2 lv;
          lv.x = *reinterpret_cast<const uint32_t*>(&l0);
          lv.y = *reinterpret_cast<const uint32_t*>(&l1);
          *reinterpret_cast<uint2*>(prod_lo + at) = lv;
        }
      }
    });
  }
}

// The same for 48 channels with one thread per sample.  Consecutive list entries are samples of
// neighbouring rays at the same rank (see the order of the appearance list), so the 32 lanes of a
// load read a few texels between them, and their rows in the tile are consecutive: every store
// instruction writes 512 contiguous bytes.  With fp32 storage a thread takes the 48 channels of a
// pair in six rounds of 8: six 256-bit loads, the fp32 interpolation and product of
// pair_products_tap, and one 16-byte store, which is exactly one k group of its row (fp16 storage:
// pair_products_thread48_h2 below).
constexpr int kThreadBlock = 128;

template <bool HALF>
__device__ __forceinline__ void load8(const void* base, uint32_t texel, int h, float4& lo, float4& hi) {
  if constexpr (HALF) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(base) + (size_t)texel * 96u) + h);
    const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&a.x)), a1 = __half22float2(*reinterpret_cast<const __half2*>(&a.y));
    const float2 a2 = __half22float2(*reinterpret_cast<const __half2*>(&a.z)), a3 = __half22float2(*reinterpret_cast<const __half2*>(&a.w));
    lo = make_float4(a0.x, a0.y, a1.x, a1.y);
    hi = make_float4(a2.x, a2.y, a3.x, a3.y);
  } else {
    const F8 v = ldg8(reinterpret_cast<const float*>(base) + (size_t)texel * 48u + 8 * h);
    lo = v.lo;
    hi = v.hi;
  }
}

template <bool HALF>
__device__ __forceinline__ void pair_products_thread48(const GnrPlane& pl, Tap tx, Tap ty, Tap tl, unsigned char* out) {
  const float ax1 = tx.f1, ay1 = ty.f1, al1 = tl.f1;
  const float ax0 = 1.0f - ax1, ay0 = 1.0f - ay1, al0 = 1.0f - al1;
  const float w_nw = ax0 * ay0, w_ne = ax1 * ay0, w_sw = ax0 * ay1, w_se = ax1 * ay1;
  const uint32_t nw = (uint32_t)ty.i0 * (uint32_t)pl.W + (uint32_t)tx.i0, sw = nw + (uint32_t)pl.W;
  const uint32_t seg = (uint32_t)tl.i0;
#pragma unroll
  for (int h = 0; h < 6; ++h) {
    float4 nwl, nwh, nel, neh, swl, swh, sel, seh, l0l, l0h, l1l, l1h;
    load8<HALF>(pl.plane, nw, h, nwl, nwh);
    load8<HALF>(pl.plane, nw + 1u, h, nel, neh);
    load8<HALF>(pl.plane, sw, h, swl, swh);
    load8<HALF>(pl.plane, sw + 1u, h, sel, seh);
    load8<HALF>(pl.line, seg, h, l0l, l0h);
    load8<HALF>(pl.line, seg + 1u, h, l1l, l1h);
    float4 pa = f4_scale(nwl, w_nw), pb = f4_scale(nwh, w_nw);
    pa = f4_fma(nel, w_ne, pa);
    pb = f4_fma(neh, w_ne, pb);
    pa = f4_fma(swl, w_sw, pa);
    pb = f4_fma(swh, w_sw, pb);
    pa = f4_fma(sel, w_se, pa);
    pb = f4_fma(seh, w_se, pb);
    const float4 la = f4_fma(l1l, al1, f4_scale(l0l, al0)), lb = f4_fma(l1h, al1, f4_scale(l0h, al0));
    const float4 qa = f4_mul(pa, la), qb = f4_mul(pb, lb);
    const __half2 h0 = __floats2half2_rn(qa.x, qa.y), h1 = __floats2half2_rn(qa.z, qa.w);
    const __half2 h2 = __floats2half2_rn(qb.x, qb.y), h3 = __floats2half2_rn(qb.z, qb.w);
    uint4 v;
    v.x = *reinterpret_cast<const uint32_t*>(&h0);
    v.y = *reinterpret_cast<const uint32_t*>(&h1);
    v.z = *reinterpret_cast<const uint32_t*>(&h2);
    v.w = *reinterpret_cast<const uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(out + (size_t)h * 2048) = v;
  }
}

__device__ __forceinline__ void pair_products_thread48_h2(const GnrPlane& pl, Tap tx, Tap ty, Tap tl, unsigned char* out) {
  const PairTapsH2 t = make_pair_taps_h2(pl, tx, ty, tl);
#pragma unroll
  for (int g = 0; g < 3; ++g) {
    uint32_t q[8];
    pair_round_h2(pl, t, g, q);
    *reinterpret_cast<uint4*>(out + (size_t)(2 * g) * 2048) = make_uint4(q[0], q[1], q[2], q[3]);
    *reinterpret_cast<uint4*>(out + (size_t)(2 * g + 1) * 2048) = make_uint4(q[4], q[5], q[6], q[7]);
  }
}

template <int NP, bool HALF>
__global__ void __launch_bounds__(kThreadBlock, 4)
app_products_thread_kernel(GnrSampleParams p, PlaneSet planes, GnrCoords crd, unsigned char* __restrict__ prod_hi,
                           int tile_bytes, int view_group) {
  const long long total = coords_total(crd);
  // contiguous share of the list per CTA, in steps of kThreadBlock entries
  const long long steps = (total + kThreadBlock - 1) / kThreadBlock;
  const long long per = (steps + gridDim.x - 1) / gridDim.x;
  const long long range_beg = min(total, (long long)blockIdx.x * per * kThreadBlock);
  const long long range_end = min(total, range_beg + per * kThreadBlock);
  for (long long j = range_beg + threadIdx.x; j < range_end; j += kThreadBlock) {
    float x, y, z, view[3];
    sample_xyz(p, crd, j, x, y, z, view);
    unsigned char* row = prod_hi + (size_t)(j >> 7) * tile_bytes + (size_t)(j & 127) * 16;
    {
      const __half hx = __float2half_rn(view[0]), hy = __float2half_rn(view[1]), hz = __float2half_rn(view[2]);
      const __half2 a = __halves2half2(hx, hy);
      const __half2 b = __halves2half2(hz, __float2half_rn(view[0] - __half2float(hx)));
      const __half2 c = __floats2half2_rn(view[1] - __half2float(hy), view[2] - __half2float(hz));
      uint4 vv;
      vv.x = *reinterpret_cast<const uint32_t*>(&a);
      vv.y = *reinterpret_cast<const uint32_t*>(&b);
      vv.z = *reinterpret_cast<const uint32_t*>(&c);
      vv.w = 0u;
      *reinterpret_cast<uint4*>(row + (size_t)view_group * 2048) = vv;
    }
    if (NP == 3) {
      const Tap tx = make_tap(x, planes.p[0].fw, planes.p[0].W);
      const Tap ty = make_tap(y, planes.p[0].fh, planes.p[0].H);
      const Tap tz = make_tap(z, planes.p[0].fl, planes.p[0].L);
      if constexpr (HALF) {
        pair_products_thread48_h2(planes.p[0], tx, ty, tz, row);
        pair_products_thread48_h2(planes.p[1], tx, tz, ty, row + 6 * 2048);
        pair_products_thread48_h2(planes.p[2], ty, tz, tx, row + 12 * 2048);
      } else {
        pair_products_thread48<HALF>(planes.p[0], tx, ty, tz, row);
        pair_products_thread48<HALF>(planes.p[1], tx, tz, ty, row + 6 * 2048);
        pair_products_thread48<HALF>(planes.p[2], ty, tz, tx, row + 12 * 2048);
      }
    } else {
      for (int pi = 0; pi < planes.n; ++pi) {
        const GnrPlane& pl = planes.p[pi];
        const float u = pick(x, y, z, pl.mat0), v = pick(x, y, z, pl.mat1), l = pick(x, y, z, pl.vec);
        const Tap tu = make_tap(u, pl.fw, pl.W), tv = make_tap(v, pl.fh, pl.H), tl = make_tap(l, pl.fl, pl.L);
        if constexpr (HALF) pair_products_thread48_h2(pl, tu, tv, tl, row + (size_t)pi * 6 * 2048);
        else pair_products_thread48<HALF>(pl, tu, tv, tl, row + (size_t)pi * 6 * 2048);
      }
    }
  }
}

// Normalised positions (and ray numbers) of the valid samples, for renderers that route
// samples to the GPU that owns their part of the field.
__global__ void positions_kernel(GnrSampleParams p, GnrCoords crd, float* __restrict__ xyz, int32_t* __restrict__ ray_index) {
  const long long total = coords_total(crd);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    float x, y, z;
    sample_xyz(p, crd, i, x, y, z);
    xyz[i * 3 + 0] = x;
    xyz[i * 3 + 1] = y;
    xyz[i * 3 + 2] = z;
    if (ray_index) ray_index[i] = (int32_t)(__ldg(crd.ids + i) >> p.kbits);
  }
}

}  // namespace

GnrCoords gnr_coords_valid(const float* rays, char* ws, const GnrWs& L) {
  GnrCoords c;
  c.rays = rays;
  c.t_min = (const float*)(ws + L.t_min);
  c.ids = (const uint32_t*)(ws + L.ids);
  c.index = nullptr;
  c.xyz_direct = nullptr;
  c.view_direct = nullptr;
  c.point_stride = 3;
  c.blk_px = c.blk_py = c.blk_bx = c.blk_by = 0;
  c.blk_pw = c.blk_ph = 0.0f;
  c.total_ptr = (const int32_t*)(ws + L.offsets) + L.n_rays;
  c.total_direct = 0;
  c.capacity = L.max_valid;
  return c;
}

GnrCoords gnr_coords_app(const float* rays, char* ws, const GnrWs& L) {
  GnrCoords c = gnr_coords_valid(rays, ws, L);
  c.ids = (const uint32_t*)(ws + L.app_ids);  // written by expand_app_kernel in list order
  c.total_ptr = (const int32_t*)(ws + L.app_offsets) + L.n_rays;
  c.capacity = L.max_app;
  return c;
}

// ---- measurement helper: rate of L1-resident 256-bit loads ------------------------------------------
// Every warp re-reads its own 8 KB window (1 KB per instruction, lanes 32 bytes apart) of a per-CTA
// buffer that stays in L1: what the kernel moves is exactly the L1 -> register traffic the gathers are
// bound by, with no misses, no address arithmetic to speak of and eight loads in flight per thread.
namespace {
__global__ void __launch_bounds__(256) l1_read_kernel(const float* __restrict__ buf, int iters, float* __restrict__ sink) {
  const float* base = buf + (size_t)blockIdx.x * 16384 + (threadIdx.x >> 5) * 2048 + (threadIdx.x & 31) * 8;
  float acc = 0.0f;
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      // volatile: every iteration really loads (the window is re-read, it never changes)
      float a0, a1, a2, a3, a4, a5, a6, a7;
      asm volatile("ld.global.nc.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                   : "=f"(a0), "=f"(a1), "=f"(a2), "=f"(a3), "=f"(a4), "=f"(a5), "=f"(a6), "=f"(a7)
                   : "l"(base + ((u + it) & 7) * 256));  // the address depends on `it`: nothing can be hoisted
      acc += (a0 + a1) + (a2 + a3) + (a4 + a5) + (a6 + a7);
    }
  }
  if (acc == 123.456f) sink[0] = acc;  // never true for the zero-filled buffer; keeps the sums alive
}
}  // namespace

extern "C" int gnr_measure_l1_bandwidth(int device, int iters, float* gb_per_s_h) {
  if (!gb_per_s_h || iters < 1 || iters > (1 << 20)) {
    gnr_set_error("gnr_measure_l1_bandwidth: bad argument");
    return -1;
  }
  int prev = 0;
  cudaGetDevice(&prev);
  GNR_CUDA_OK(cudaSetDevice(device));
  cudaDeviceProp prop;
  GNR_CUDA_OK(cudaGetDeviceProperties(&prop, device));
  const int ctas = prop.multiProcessorCount * 4;
  float *buf = nullptr, *sink = nullptr;
  cudaEvent_t e0, e1;
  GNR_CUDA_OK(cudaMalloc(&buf, (size_t)ctas * 16384 * sizeof(float)));
  GNR_CUDA_OK(cudaMalloc(&sink, 256));
  GNR_CUDA_OK(cudaMemset(buf, 0, (size_t)ctas * 16384 * sizeof(float)));
  GNR_CUDA_OK(cudaEventCreate(&e0));
  GNR_CUDA_OK(cudaEventCreate(&e1));
  l1_read_kernel<<<ctas, 256>>>(buf, 16, sink);  // warm-up
  GNR_CUDA_OK(cudaEventRecord(e0));
  l1_read_kernel<<<ctas, 256>>>(buf, iters, sink);
  GNR_CUDA_OK(cudaEventRecord(e1));
  GNR_CUDA_OK(cudaEventSynchronize(e1));
  float ms = 0.0f;
  GNR_CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
  *gb_per_s_h = (float)((double)ctas * 256 * iters * 8 * 32 / (ms * 1e-3) / 1e9);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(buf);
  cudaFree(sink);
  cudaSetDevice(prev);
  return 0;
}

static LatticeRef lattice_of(const GnrModel* m) {
  LatticeRef r;
  r.v = m->den_lattice;
  r.gx = m->lat_dims[0];
  r.gy = m->lat_dims[1];
  r.gz = m->lat_dims[2];
  return r;
}

int launch_build_lattice(const GnrModel* m, float* V, cudaStream_t st) {
  PlaneSet set = make_set(m->den, m->cfg.n_pairs);
  if (!standard_vm3(set)) {
    gnr_set_error("the density lattice needs the standard three-pair layout on one grid (xy|z, xz|y, yz|x)");
    return -1;
  }
  const int gx = set.p[0].W, gy = set.p[0].H, gz = set.p[0].L;
  const int grid = m->sm_count * 16;
  if (m->cfg.den_storage == 1)
    build_lattice_kernel<true><<<grid, 256, 0, st>>>(set, set.p[0].C, gx, gy, gz, V);
  else
    build_lattice_kernel<false><<<grid, 256, 0, st>>>(set, set.p[0].C, gx, gy, gz, V);
  return (int)cudaGetLastError();
}

int gnr_app_lattice_dims(const GnrModel* m, int* dims) {
  PlaneSet set = make_set(m->app, m->cfg.n_pairs);
  for (int i = 0; i < m->cfg.n_pairs; ++i) {
    if (!m->app[i].plane || !m->app[i].line) {
      gnr_set_error("appearance plane/line pair %d has not been uploaded", i);
      return -1;
    }
  }
  if (!standard_vm3(set) || set.p[0].C != 48 || m->cfg.app_dim > 27 || !m->mlp.basis_raw) {
    gnr_set_error("the appearance lattice needs the standard three-pair layout on one grid, 33..48 appearance channels, "
                  "app_dim <= 27 and uploaded MLP weights");
    return -1;
  }
  dims[0] = set.p[0].W;
  dims[1] = set.p[0].H;
  dims[2] = set.p[0].L;
  return 0;
}

int launch_build_app_lattice(const GnrModel* m, void* V, cudaStream_t st) {
  PlaneSet set = make_set(m->app, m->cfg.n_pairs);
  const int gx = set.p[0].W, gy = set.p[0].H, gz = set.p[0].L;
  const size_t smem = 3 * 48 * 28 * sizeof(float);
  const int grid = m->sm_count * 16;
  if (m->cfg.app_storage == 1)
    build_app_lattice_kernel<true><<<grid, 128, smem, st>>>(set, m->mlp.basis_raw, m->cfg.app_dim, m->cfg.n_app, gx, gy, gz, (__half*)V);
  else
    build_app_lattice_kernel<false><<<grid, 128, smem, st>>>(set, m->mlp.basis_raw, m->cfg.app_dim, m->cfg.n_app, gx, gy, gz, (__half*)V);
  return (int)cudaGetLastError();
}

int gnr_lattice_dims(const GnrModel* m, int* dims) {
  PlaneSet set = make_set(m->den, m->cfg.n_pairs);
  for (int i = 0; i < m->cfg.n_pairs; ++i) {
    if (!m->den[i].plane || !m->den[i].line) {
      gnr_set_error("density plane/line pair %d has not been uploaded", i);
      return -1;
    }
  }
  if (!standard_vm3(set)) {
    gnr_set_error("the density lattice needs the standard three-pair layout on one grid (xy|z, xz|y, yz|x)");
    return -1;
  }
  dims[0] = set.p[0].W;
  dims[1] = set.p[0].H;
  dims[2] = set.p[0].L;
  if ((long long)dims[0] * dims[1] * dims[2] > 0xffffffffLL) {
    gnr_set_error("density lattice of %dx%dx%d points exceeds 32-bit offsets", dims[0], dims[1], dims[2]);
    return -1;
  }
  return 0;
}

int launch_density(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, float* sigma_feat, float* sigma,
                   cudaStream_t st) {
  PlaneSet set = make_set(m->den, m->cfg.n_pairs);
  const int J = m->den[0].C / 16;
  const int grid = m->sm_count * 4;
  if (m->den_lattice) {
    density_lattice_kernel<<<m->sm_count * 8, kBlock, 0, st>>>(p, set, lattice_of(m), c, m->cfg.density_shift, m->cfg.density_act,
                                                              sigma_feat, sigma);
    return (int)cudaGetLastError();
  }
#define GNR_DEN(JJ)                                                                                                   \
  do {                                                                                                                \
    if (standard_vm3(set))                                                                                            \
      density_kernel<JJ, 3><<<grid, kBlock, 0, st>>>(p, set, c, m->cfg.density_shift, m->cfg.density_act, sigma_feat, sigma); \
    else                                                                                                              \
      density_kernel<JJ, 0><<<grid, kBlock, 0, st>>>(p, set, c, m->cfg.density_shift, m->cfg.density_act, sigma_feat, sigma); \
  } while (0)
  if (m->cfg.den_storage == 1) {  // fp16 planes: 16 channels (checked at creation)
    if (standard_vm3(set))
      density_kernel<1, 3, true><<<grid, kBlock, 0, st>>>(p, set, c, m->cfg.density_shift, m->cfg.density_act, sigma_feat, sigma);
    else
      density_kernel<1, 0, true><<<grid, kBlock, 0, st>>>(p, set, c, m->cfg.density_shift, m->cfg.density_act, sigma_feat, sigma);
    return (int)cudaGetLastError();
  }
  switch (J) {
    case 1: GNR_DEN(1); break;
    case 2: GNR_DEN(2); break;
    case 3: GNR_DEN(3); break;
    case 4: GNR_DEN(4); break;
    default: gnr_set_error("density channels (padded) %d not supported (16..64)", m->den[0].C); return -1;
  }
#undef GNR_DEN
  return (int)cudaGetLastError();
}

int launch_app_gather(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, int feat_stride, float* feat,
                      cudaStream_t st) {
  if (m->cfg.app_storage != 0) {
    gnr_set_error("the CUDA-core appearance gather reads fp32 planes; this model holds them as fp16 (app_storage 1)");
    return -1;
  }
  PlaneSet set = make_set(m->app, m->cfg.n_pairs);
  const int J = m->app[0].C / 16;
  const int grid = m->sm_count * 4;
  size_t smem = (size_t)m->cfg.n_pairs * 4 * (4 * J * kFeat + 8) * sizeof(float);
#define GNR_APP(JJ)                                                                                            \
  do {                                                                                                         \
    cudaFuncSetAttribute(app_gather_kernel<JJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
    app_gather_kernel<JJ><<<grid, kBlock, smem, st>>>(p, set, c, m->mlp.basis_blocked, feat_stride, feat);     \
  } while (0)
  switch (J) {
    case 1: GNR_APP(1); break;
    case 2: GNR_APP(2); break;
    case 3: GNR_APP(3); break;
    case 4: GNR_APP(4); break;
    default: gnr_set_error("appearance channels (padded) %d not supported (16..64)", m->app[0].C); return -1;
  }
#undef GNR_APP
  return (int)cudaGetLastError();
}

int launch_app_products(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, unsigned char* hi,
                        unsigned char* lo, int tile_bytes, int terms, cudaStream_t st) {
  PlaneSet set = make_set(m->app, m->cfg.n_pairs);
  const int J = m->app[0].C / 16;
  const int grid = m->sm_count * 4;
#define GNR_PRD(JJ, NPP, TT) app_products_kernel<JJ, NPP, TT><<<grid, kBlock, 0, st>>>(p, set, c, hi, lo, tile_bytes, m->mlp.n_prod / 8)
  if (m->cfg.app_storage == 1 && (J != 3 || terms != 1)) {
    gnr_set_error("fp16 appearance planes need 48 (padded) channels and mlp_mode 2");
    return -1;
  }
  if (J == 3 && terms == 1 && m->cfg.app_storage == 1) {
    // fp16 storage: one thread per sample; fp32 storage below: four lanes per sample, which the L1
    // serves better when every load instruction moves 16 bytes per lane
    const int tgrid = m->sm_count * 8;
    const bool vm3 = standard_vm3(set), half = m->cfg.app_storage == 1;
#define GNR_PRT(NPP, HH) \
  app_products_thread_kernel<NPP, HH><<<tgrid, kThreadBlock, 0, st>>>(p, set, c, hi, tile_bytes, m->mlp.n_prod / 8)
    if (vm3 && half) GNR_PRT(3, true);
    else if (vm3) GNR_PRT(3, false);
    else if (half) GNR_PRT(0, true);
    else GNR_PRT(0, false);
#undef GNR_PRT
  } else if (J == 3 && standard_vm3(set)) {
    if (terms == 2) GNR_PRD(3, 3, 2); else GNR_PRD(3, 3, 1);
  } else if (J == 1) {
    if (terms == 2) GNR_PRD(1, 0, 2); else GNR_PRD(1, 0, 1);
  } else if (J == 2) {
    if (terms == 2) GNR_PRD(2, 0, 2); else GNR_PRD(2, 0, 1);
  } else if (J == 3) {
    if (terms == 2) GNR_PRD(3, 0, 2); else GNR_PRD(3, 0, 1);
  } else {
    gnr_set_error("appearance channels (padded) %d not supported by the tensor-core path", m->app[0].C);
    return -1;
  }
#undef GNR_PRD
  return (int)cudaGetLastError();
}

int launch_positions(const GnrModel* m, const GnrSampleParams& p, const GnrCoords& c, float* xyz, int32_t* ray_index,
                     cudaStream_t st) {
  positions_kernel<<<m->sm_count * 8, 256, 0, st>>>(p, c, xyz, ray_index);
  return (int)cudaGetLastError();
}

int launch_march(const GnrModel* m, const GnrSampleParams& p, const float* rays, int64_t n, char* ws, const GnrWs& L,
                 cudaStream_t st, int list_only) {
  PlaneSet set = make_set(m->den, m->cfg.n_pairs);
  const int J = m->den[0].C / 16;
  const unsigned grid = (unsigned)((n + kMarchBlock - 1) / kMarchBlock);
  const float t_stop = m->cfg.ert_transmittance > 0.0f ? m->cfg.ert_transmittance : 0.0f;
  const LatticeRef lat = lattice_of(m);
#define GNR_MARCH(JJ, NPP) GNR_MARCH_H(JJ, NPP, false, false)
#define GNR_MARCH_H(JJ, NPP, HH, LL)                                                                              \
  march_kernel<JJ, NPP, HH, LL><<<grid, kMarchBlock, 0, st>>>(                                                    \
      p, set, lat, rays, (const float*)(ws + L.t_min), (const uint32_t*)(ws + L.words), (const int32_t*)(ws + L.offsets), \
      (long long)n, L.max_valid, m->cfg.density_shift, m->cfg.density_act, m->cfg.distance_scale,                 \
      m->cfg.ray_weight_thres, t_stop, (float*)(ws + L.weight), (float*)(ws + L.acc), (float*)(ws + L.depth),     \
      (int32_t*)(ws + L.app_counts), (int32_t*)(ws + L.status) + GNR_ST_NUM_DENSITY, list_only, (float2*)(ws + L.sigma))
  if (m->den_lattice) GNR_MARCH_H(1, 3, false, true);
  else if (m->cfg.den_storage == 1 && standard_vm3(set)) GNR_MARCH_H(1, 3, true, false);
  else if (m->cfg.den_storage == 1) GNR_MARCH_H(1, 0, true, false);
  else if (J == 1 && standard_vm3(set)) GNR_MARCH(1, 3);
  else if (J == 1) GNR_MARCH(1, 0);
  else if (J == 2) GNR_MARCH(2, 0);
  else if (J == 3) GNR_MARCH(3, 0);
  else if (J == 4) GNR_MARCH(4, 0);
  else {
    gnr_set_error("density channels (padded) %d not supported (16..64)", m->den[0].C);
    return -1;
  }
#undef GNR_MARCH
#undef GNR_MARCH_H
  return (int)cudaGetLastError();
}
