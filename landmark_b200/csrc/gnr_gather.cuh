// Pieces of the VM feature gather that more than one translation unit uses: the plane-set
// argument, the tap arithmetic, the position of a list entry, and the packed-fp16 interpolation of
// one plane/line pair (48 channels from fp16 storage).
#pragma once
#include <cuda_fp16.h>

#include "gnr_internal.cuh"

namespace {

struct PlaneSet {
  GnrPlane p[GNR_MAX_PLANES];
  int n;
};

__device__ __forceinline__ float pick(float x, float y, float z, int a) { return a == 0 ? x : (a == 1 ? y : z); }

// Lower grid index and fractional offset of one normalised coordinate on an axis of `size` points.
struct Tap {
  int i0;
  float f1;
};
__device__ __forceinline__ Tap make_tap(float u, float fsize, int size) {
  const float ix = fminf(fmaxf((u + 1.0f) * 0.5f * fsize, 0.0f), fsize);
  Tap t;
  t.i0 = min((int)ix, size - 2);
  t.f1 = ix - (float)t.i0;
  return t;
}

// Coordinates of a normalised position inside block (bx, by) of a division into blocks of width pw x ph: the
// arithmetic of assign_blocks_to_samples (app/models/gridnerf_parallel.py:296-327), one rounded fp32 operation per
// step in torch's order: coord_min = -1 + b * width, coord_max = -1 + (b + 1) * width,
// local = (p - min) * 2 / (max - min) - 1.
__device__ __forceinline__ void block_local(float bx, float by, float pw, float ph, float x, float y, float& lx, float& ly) {
  const float x0 = __fadd_rn(-1.0f, __fmul_rn(bx, pw)), x1 = __fadd_rn(-1.0f, __fmul_rn(__fadd_rn(bx, 1.0f), pw));
  const float y0 = __fadd_rn(-1.0f, __fmul_rn(by, ph)), y1 = __fadd_rn(-1.0f, __fmul_rn(__fadd_rn(by, 1.0f), ph));
  lx = __fsub_rn(__fdiv_rn(__fmul_rn(__fsub_rn(x, x0), 2.0f), __fsub_rn(x1, x0)), 1.0f);
  ly = __fsub_rn(__fdiv_rn(__fmul_rn(__fsub_rn(y, y0), 2.0f), __fsub_rn(y1, y0)), 1.0f);
}

// Normalised position of item i.  List mode: recomputed from the ray exactly as the sampler
// computed it, then normalised as normalize_coord does (app/models/gridnerf_sequential.py:203-204).
// `view` (optional) receives the ray direction of the sample.
__device__ __forceinline__ void sample_xyz(const GnrSampleParams& p, const GnrCoords& c, long long i, float& x, float& y,
                                           float& z, float* view = nullptr) {
  if (c.xyz_direct) {
    const long long at = i * c.point_stride;
    x = __ldg(c.xyz_direct + at + 0);
    y = __ldg(c.xyz_direct + at + 1);
    z = __ldg(c.xyz_direct + at + 2);
    if (view) {
#pragma unroll
      for (int a = 0; a < 3; ++a) view[a] = c.view_direct ? __ldg(c.view_direct + at + a) : 0.0f;
    }
    return;
  }
  const uint32_t id = __ldg(c.ids + (c.index ? (long long)__ldg(c.index + i) : i));
  const uint32_t ray = id >> p.kbits;
  const int k = (int)(id & ((1u << p.kbits) - 1u));
  const float* r = c.rays + (size_t)ray * 6;
  const float t = gnr_sample_t(p, __ldg(c.t_min + ray), k);
  const float dx = __ldg(r + 3), dy = __ldg(r + 4), dz = __ldg(r + 5);
  x = gnr_normalize(gnr_point(__ldg(r + 0), dx, t), p.lo[0], p.inv[0]);
  y = gnr_normalize(gnr_point(__ldg(r + 1), dy, t), p.lo[1], p.inv[1]);
  z = gnr_normalize(gnr_point(__ldg(r + 2), dz, t), p.lo[2], p.inv[2]);
  if (c.blk_px > 0) block_local((float)c.blk_bx, (float)c.blk_by, c.blk_pw, c.blk_ph, x, y, x, y);
  if (view) {
    view[0] = dx;
    view[1] = dy;
    view[2] = dz;
  }
}

__device__ __forceinline__ long long coords_total(const GnrCoords& c) {
  const long long t = c.total_ptr ? (long long)*c.total_ptr : c.total_direct;
  return min(t, c.capacity);
}

// fp16 storage: the 48 channels of a pair in three rounds of 16, six 256-bit loads per round, and
// the interpolation itself in packed fp16 arithmetic (two channels per instruction, no
// conversions).  Against fp32 interpolation of the same fp16 texels this adds four more fp16
// roundings to a product that is rounded to fp16 for the tensor cores anyway; the rounding of
// the stored texels remains the larger part of the error of the projected features.
struct H16 {
  uint32_t v[8];
};
__device__ __forceinline__ H16 ldg_h16(const void* base, uint32_t texel, int g) {
  const unsigned char* ptr = reinterpret_cast<const unsigned char*>(base) + (size_t)texel * 96u + g * 32;
  H16 r;
  asm("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7])
      : "l"(ptr));
  return r;
}
__device__ __forceinline__ __half2 as_h2(uint32_t u) { return *reinterpret_cast<const __half2*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<const uint32_t*>(&h); }

// Interpolation weights and texel numbers of one pair for one sample.
struct PairTapsH2 {
  __half2 w_nw, w_ne, w_sw, w_se, h_l0, h_l1;
  uint32_t nw, sw, seg;
};
__device__ __forceinline__ PairTapsH2 make_pair_taps_h2(const GnrPlane& pl, Tap tx, Tap ty, Tap tl) {
  const float ax1 = tx.f1, ay1 = ty.f1, al1 = tl.f1;
  const float ax0 = 1.0f - ax1, ay0 = 1.0f - ay1, al0 = 1.0f - al1;
  PairTapsH2 t;
  t.w_nw = __float2half2_rn(ax0 * ay0);
  t.w_ne = __float2half2_rn(ax1 * ay0);
  t.w_sw = __float2half2_rn(ax0 * ay1);
  t.w_se = __float2half2_rn(ax1 * ay1);
  t.h_l0 = __float2half2_rn(al0);
  t.h_l1 = __float2half2_rn(al1);
  t.nw = (uint32_t)ty.i0 * (uint32_t)pl.W + (uint32_t)tx.i0;
  t.sw = t.nw + (uint32_t)pl.W;
  t.seg = (uint32_t)tl.i0;
  return t;
}
// Channels 16 g .. 16 g + 15 of the pair's plane x line products as eight packed fp16 pairs:
// q[e] = channels 16 g + 2 e (low half) and 16 g + 2 e + 1.
__device__ __forceinline__ void pair_round_h2(const GnrPlane& pl, const PairTapsH2& t, int g, uint32_t (&q)[8]) {
  const H16 a = ldg_h16(pl.plane, t.nw, g), b = ldg_h16(pl.plane, t.nw + 1u, g);
  const H16 c = ldg_h16(pl.plane, t.sw, g), d = ldg_h16(pl.plane, t.sw + 1u, g);
  const H16 l0 = ldg_h16(pl.line, t.seg, g), l1 = ldg_h16(pl.line, t.seg + 1u, g);
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

// True if the three pairs are the standard VM layout on one grid: (x,y|z), (x,z|y), (y,z|x).
bool standard_vm3(const PlaneSet& s) {
  if (s.n != 3) return false;
  const GnrPlane &a = s.p[0], &b = s.p[1], &c = s.p[2];
  const bool modes = a.mat0 == 0 && a.mat1 == 1 && a.vec == 2 && b.mat0 == 0 && b.mat1 == 2 && b.vec == 1 &&
                     c.mat0 == 1 && c.mat1 == 2 && c.vec == 0;
  const bool sizes = b.W == a.W && b.H == a.L && b.L == a.H && c.W == a.H && c.H == a.L && c.L == a.W;
  return modes && sizes;
}

PlaneSet make_set(const GnrPlane* src, int n) {
  PlaneSet s;
  s.n = n;
  for (int i = 0; i < n; ++i) s.p[i] = src[i];
  return s;
}

}  // namespace
