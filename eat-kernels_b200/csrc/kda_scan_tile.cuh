// One step of a scan of affine state maps on a register-tiled block:  E <- E P + L  for 32 independent rows of one
// head (fp32 throughout, the products summed in the order k = 0 .. 127 on top of L, whatever the tiling).
//
// 256 threads carry a [32][128] block of E as 4x4 register tiles (thread (ty, tx): rows 4 ty .. 4 ty + 3, columns
// 4 tx .. 4 tx + 3).  Per step the block is published transposed in shared memory (so the four rows of a thread at one
// k are one 16-byte broadcast load) and P streams through a double-buffered [16][128] slice: 2 shared loads per 16
// multiply-adds, against 5 loads per 4 when every thread carries a single row.  P is read once per CTA and step (four
// CTAs per head), coalesced.
#pragma once
#include "kda_common.cuh"

namespace kda {

constexpr int ST_ROWS = 32, ST_THREADS = 256, ST_KSLICE = 16;

struct ScanSmem {
  float sT[D][ST_ROWS];                 // E transposed: [k][row]
  float sP[2][ST_KSLICE][D];            // slices of P
};

// Element (r, k) of a state sits at r * rs + k * ks: (D, 1) in the value-first layout (rows = values), (1, D) when the
// independent index is the contiguous one (key-first states: columns evolve independently).  One of the two is 1, so a
// thread's 4x4 tile is four 16-byte accesses either way.
__device__ __forceinline__ void scan_tile_load(float (&t)[4][4], const float* base, int r0, int c0, int ks) {
  if (ks == 1) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float4 f = *reinterpret_cast<const float4*>(base + (size_t)(r0 + i) * D + c0);
      t[i][0] = f.x; t[i][1] = f.y; t[i][2] = f.z; t[i][3] = f.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float4 f = *reinterpret_cast<const float4*>(base + (size_t)(c0 + j) * D + r0);
      t[0][j] = f.x; t[1][j] = f.y; t[2][j] = f.z; t[3][j] = f.w;
    }
  }
}

__device__ __forceinline__ void scan_tile_store(const float (&t)[4][4], float* base, int r0, int c0, int ks) {
  if (ks == 1) {
#pragma unroll
    for (int i = 0; i < 4; i++)
      *reinterpret_cast<float4*>(base + (size_t)(r0 + i) * D + c0) = make_float4(t[i][0], t[i][1], t[i][2], t[i][3]);
  } else {
#pragma unroll
    for (int j = 0; j < 4; j++)
      *reinterpret_cast<float4*>(base + (size_t)(c0 + j) * D + r0) = make_float4(t[0][j], t[1][j], t[2][j], t[3][j]);
  }
}

// acc holds the L tile on entry and E P + L on exit; cur is the thread's tile of E; Pi is the head's map [128][128]
// (value-first: row k, column k').  Every thread of the CTA calls this.
__device__ __forceinline__ void scan_tile_step(float (&acc)[4][4], const float (&cur)[4][4], const float* __restrict__ Pi,
                                               ScanSmem& sm, int tid) {
  const int ty = tid >> 5, tx = tid & 31;
  const float4* P4 = reinterpret_cast<const float4*>(Pi);
  float4 pa = P4[tid], pb = P4[tid + ST_THREADS];                        // slice 0: rows 0-7 and 8-15
  __syncthreads();                                                       // the previous step's readers are done
#pragma unroll
  for (int j = 0; j < 4; j++)
    *reinterpret_cast<float4*>(&sm.sT[4 * tx + j][4 * ty]) = make_float4(cur[0][j], cur[1][j], cur[2][j], cur[3][j]);
  *reinterpret_cast<float4*>(&sm.sP[0][ty][4 * tx]) = pa;
  *reinterpret_cast<float4*>(&sm.sP[0][8 + ty][4 * tx]) = pb;
  __syncthreads();
#pragma unroll 1
  for (int s = 0; s < D / ST_KSLICE; s++) {
    if (s + 1 < D / ST_KSLICE) {
      pa = P4[(s + 1) * (ST_KSLICE * D / 4) + tid];
      pb = P4[(s + 1) * (ST_KSLICE * D / 4) + tid + ST_THREADS];
    }
#pragma unroll
    for (int kk = 0; kk < ST_KSLICE; kk++) {
      const float4 e = *reinterpret_cast<const float4*>(&sm.sT[s * ST_KSLICE + kk][4 * ty]);
      const float4 p = *reinterpret_cast<const float4*>(&sm.sP[s & 1][kk][4 * tx]);
      const float ev[4] = {e.x, e.y, e.z, e.w}, pv[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(ev[i], pv[j], acc[i][j]);
    }
    if (s + 1 < D / ST_KSLICE) {
      *reinterpret_cast<float4*>(&sm.sP[(s + 1) & 1][ty][4 * tx]) = pa;
      *reinterpret_cast<float4*>(&sm.sP[(s + 1) & 1][8 + ty][4 * tx]) = pb;
    }
    __syncthreads();
  }
}

}  // namespace kda
