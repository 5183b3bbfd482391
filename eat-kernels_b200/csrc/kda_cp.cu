// Context parallelism over token segments (within one GPU or across GPUs) and state row copies.
//
// The recurrence is affine in the state, so a segment that does not yet know its entering state S_in can still run:
// chain L from S = 0 gives (o_loc, S_loc), chain Tr from S = I with v = 0 gives (Qt, P), and afterwards
//     S_end = S_in @ P + S_loc          out_t = o_loc_t + S_in applied to Qt_t          (value-first orientation)
// (the algebra of kda/b200/csrc/w3/kernel.py:22-38 and kda/b200/csrc/w3/cp_fix.cu:4-21).  Both chains run as tasks of
// the fused chunk kernel; this file plans those tasks, scans the maps and applies the output fix-up.
#include "kda_cp.cuh"
#include "kda_scan_tile.cuh"

namespace kda {

// ------------------------------------------------------------------------------------------------ segment tasks
// Tile-major output scratch of dual-chain tasks: segment i owns ceil(len_i / 32) tiles per head, after those of the
// segments before it (every segment counts, mapped or not, so that the planner and the fix-up agree without a table).
__device__ __forceinline__ long long seg_tile0(const long long* t0s, const long long* t1s, long long T, int seg) {
  long long tiles = 0;
  for (int j = 0; j < seg; j++) {
    const long long a = max(0LL, t0s[j]), b = min(T, t1s[j]);
    if (b > a) tiles += (b - a + C - 1) / C;
  }
  return tiles;
}

__global__ void kda_seg_plan_kernel(const SegPlanParams a) {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // see kda_plan_kernel
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < a.n_seg; i += gridDim.x * blockDim.x) {
    long long t0 = a.t0[i], t1 = a.t1[i];
    if (t0 < 0) t0 = 0;
    if (t1 > a.T) t1 = a.T;
    if (t1 < t0) t1 = t0;
    const size_t slot = (size_t)i * a.H * STATE_ELEMS;
    Task l, r;
    l.t0 = t0; l.len = (int)(t1 - t0); l.flags = 0; l.src = nullptr; l.dst = a.S_loc + slot; l.ck = nullptr; l.dst2 = nullptr;
    r = l;
    if (a.need_map[i]) {
      l.flags = TF_INIT_ZERO;
      r.flags = TF_INIT_IDENTITY | TF_V_ZERO | TF_OUT_AUX;
      r.dst = a.P + slot;
      if (a.dual) {                       // both chains in one task: the map of chain Tr goes to dst2, the outputs of both
        l.flags |= TF_DUAL;               // chains to the tile-major scratch (tiles of the earlier segments come first)
        l.dst2 = a.P + slot;
        if (a.tiles != nullptr) l.ck = a.tiles + seg_tile0(a.t0, a.t1, a.T, i) * a.H * (D * C);
      }
    } else {
      if (a.src_base != nullptr) l.src = a.src_base + (size_t)i * a.src_stride;
      else l.flags = TF_INIT_ZERO;
      r.len = 0; r.flags = TF_INIT_ZERO | TF_NO_OUT; r.dst = nullptr;
    }
    if (a.no_out) {
      l.flags |= TF_NO_OUT;
      r.flags |= TF_NO_OUT;
    }
    if (a.dual) {
      a.tasks[i] = l;
    } else {
      a.tasks[2 * i] = l;
      a.tasks[2 * i + 1] = r;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *a.n_tasks = a.dual ? a.n_seg : 2 * a.n_seg;
    a.status[0] = 0; a.status[1] = 0; a.status[2] = 0; a.status[3] = 0;
  }
}

cudaError_t launch_seg_plan(const SegPlanParams& a, cudaStream_t stream) {
  kda_seg_plan_kernel<<<1, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ scan of the maps
// S_in[0] = S0 (or 0);  S_in[i+1] = S_in[i] @ P[i] + S_loc[i].  Rows of S evolve independently, so a CTA carries 32
// value rows of one head through the whole chain in fp32 as register tiles (kda_scan_tile.cuh).
__global__ void __launch_bounds__(ST_THREADS) kda_scan_kernel(const float* __restrict__ P, const float* __restrict__ S_loc,
                                                              const float* __restrict__ S0, float* __restrict__ S_in,
                                                              float* __restrict__ S_end, int n_seg, int H, long long map_stride) {
  __shared__ __align__(16) ScanSmem sm;
  const int h = blockIdx.y, tid = threadIdx.x;
  const int r0 = blockIdx.x * ST_ROWS + 4 * (tid >> 5), c0 = 4 * (tid & 31);
  const size_t head_off = (size_t)h * STATE_ELEMS;
  const size_t seg_stride = (size_t)H * STATE_ELEMS;      // of S_in; the maps may lie further apart (map_stride)
  float cur[4][4];
  if (S0 != nullptr) {
    scan_tile_load(cur, S0 + head_off, r0, c0, 1);
  } else {
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) cur[i][j] = 0.0f;
  }
  for (int i = 0; i < n_seg; i++) {
    scan_tile_store(cur, S_in + i * seg_stride + head_off, r0, c0, 1);
    float acc[4][4];
    scan_tile_load(acc, S_loc + (size_t)i * map_stride + head_off, r0, c0, 1);
    scan_tile_step(acc, cur, P + (size_t)i * map_stride + head_off, sm, tid);
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
      for (int b = 0; b < 4; b++) cur[a][b] = acc[a][b];
  }
  if (S_end != nullptr) scan_tile_store(cur, S_end + head_off, r0, c0, 1);
}

cudaError_t launch_scan(const float* P, const float* S_loc, const float* S0, float* S_in, float* S_end, int n_seg, int H,
                        long long map_stride, cudaStream_t stream) {
  dim3 grid(D / ST_ROWS, H);
  kda_scan_kernel<<<grid, ST_THREADS, 0, stream>>>(P, S_loc, S0, S_in, S_end, n_seg, H,
                                                   map_stride > 0 ? map_stride : (long long)H * STATE_ELEMS);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ output fix-up
// out[t][h][:] += bf16(S_in[seg][h]) applied to Qt[t][h][:] for the tokens of mapped segments.  A CTA owns one
// (segment, head, slice): it converts the entering state to a swizzled bf16 tile once and walks 32-token tiles.  Both
// the Qt tile and the old output tile come in through cp.async as whole 256-byte rows, the sum is formed in shared
// memory and leaves as whole rows again: the pass is pure HBM traffic (768 B per token-head), so every global access
// is a full line.
constexpr int FIX_THREADS = 256;
constexpr int FIX_SMEM = 32768 + 2 * 16384;  // bf16 state [128][128] + double-buffered {Qt tile, output tile} [32][128]

__global__ void __launch_bounds__(FIX_THREADS) kda_fixup_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ qt,
                                                                long long ldo, const float* __restrict__ S_in,
                                                                const long long* __restrict__ t0s, const long long* __restrict__ t1s,
                                                                const int* __restrict__ need_map, int n_seg, int H, int split) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slice = blockIdx.x % split;
  const int h = (blockIdx.x / split) % H;
  const int seg = blockIdx.x / (split * H);
  if (seg >= n_seg || !need_map[seg]) return;
  const long long t0 = t0s[seg], t1 = t1s[seg];
  const int ntiles = (int)((t1 - t0 + 31) / 32);
  if (slice >= ntiles) return;

  // entering state -> bf16 [v][k'] tile (row = value index: the B operand with k' contiguous)
  const float* S = S_in + ((size_t)seg * H + h) * STATE_ELEMS;
  for (int idx = tid; idx < D * D / 4; idx += FIX_THREADS) {
    const int row = idx >> 5, c4 = (idx & 31) * 4;
    const float4 f = *reinterpret_cast<const float4*>(S + row * D + c4);
    *reinterpret_cast<uint2*>(smem + tile128_off(row, c4)) = make_uint2(pack_bf16(f.x, f.y), pack_bf16(f.z, f.w));
  }
  const uint32_t s_tile = smem_u32(smem);
  const int g = lane >> 2, t = lane & 3;
  const int frag_row = 8 * (lane >> 4) + (lane & 7);
  const int frag_chunk = (lane >> 3) & 1;

  auto issue = [&](int tile, int buf) {
    const long long tok0 = t0 + (long long)tile * 32;
    const int nvalid = (int)min(32LL, t1 - tok0);
    const uint32_t dst = smem_u32(smem + 32768 + buf * 16384);
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const int idx = tid + FIX_THREADS * j, row = idx >> 4, ch = idx & 15;
      const bool ok = row < nvalid;
      const long long goff = (tok0 + (ok ? row : 0)) * ldo + (long long)h * D + ch * 8;
      const uint32_t soff = row * 256 + ((ch ^ (row & 7)) << 4);
      cp_async16(dst + soff, qt + goff, ok ? 16 : 0);
      cp_async16(dst + 8192 + soff, out + goff, ok ? 16 : 0);
    }
  };
  issue(slice, 0);
  cp_async_commit();
  int buf = 0;
  for (int tile = slice; tile < ntiles; tile += split, buf ^= 1) {
    if (tile + split < ntiles) issue(tile + split, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t q_tile = smem_u32(smem + 32768 + buf * 16384);
    uint8_t* o_tile = smem + 32768 + buf * 16384 + 8192;
    float acc[2][2][4];
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
      for (int b = 0; b < 2; b++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[a][b][c] = 0.0f;
#pragma unroll
    for (int kt = 0; kt < 8; kt++) {
      uint32_t b[4];
      ldmatrix_x4(b, s_tile + tile128_off(16 * warp + frag_row, (2 * kt + frag_chunk) * 8));
#pragma unroll
      for (int mt = 0; mt < 2; mt++) {
        uint32_t a[4];
        ldmatrix_x4(a, q_tile + tile128_off(16 * mt + (lane & 7) + ((lane >> 3) & 1) * 8, (2 * kt + (lane >> 4)) * 8));
        mma_bf16(acc[mt][0], a, b[0], b[1]);
        mma_bf16(acc[mt][1], a, b[2], b[3]);
      }
    }
    const long long tok0 = t0 + (long long)tile * 32;
    const int nvalid = (int)min(32LL, t1 - tok0);
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const int row = 16 * mt + g + 8 * half;
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
          uint32_t* o = reinterpret_cast<uint32_t*>(o_tile + tile128_off(row, 16 * warp + 8 * nt + 2 * t));
          const uint32_t old = *o;
          *o = pack_bf16(bf16_lo(old) + acc[mt][nt][2 * half], bf16_hi(old) + acc[mt][nt][2 * half + 1]);
        }
      }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const int idx = tid + FIX_THREADS * j, row = idx >> 4, ch = idx & 15;
      if (row < nvalid)
        *reinterpret_cast<uint4*>(out + (tok0 + row) * ldo + (long long)h * D + ch * 8) =
            *reinterpret_cast<const uint4*>(o_tile + row * 256 + ((ch ^ (row & 7)) << 4));
    }
    __syncthreads();
  }
}

cudaError_t launch_fixup(__nv_bfloat16* out, const __nv_bfloat16* qt, long long ldo, const float* S_in, const long long* t0,
                         const long long* t1, const int* need_map, int n_seg, int H, cudaStream_t stream) {
  static int attr_dev_mask = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(attr_dev_mask & (1 << (dev & 31)))) {
    cudaError_t e = cudaFuncSetAttribute(kda_fixup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FIX_SMEM);
    if (e != cudaSuccess) return e;
    attr_dev_mask |= 1 << (dev & 31);
  }
  int split = (16 * 148 + n_seg * H - 1) / (n_seg * H);   // about sixteen CTAs per SM: short waves, 5 % faster than four
  if (split < 1) split = 1;
  if (split > 64) split = 64;
  kda_fixup_kernel<<<(unsigned)(n_seg * H * split), FIX_THREADS, FIX_SMEM, stream>>>(out, qt, ldo, S_in, t0, t1, need_map, n_seg, H, split);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ fix-up over tiles
// The same pass for the tile-major output of dual-chain tasks: per (segment, head) and 32-token tile, the Qt tile and
// the o_loc tile are 8 KB contiguous each, [row v or k'][32 tokens] bf16.  out rows = o_loc + Qt applied to bf16(S_in).
// The Qt tile is the A operand with its rows (tokens) along the contiguous direction, so it is read with transposing
// ldmatrix; a 16-byte piece (8 tokens of one row) goes to  row * 64 + ((piece ^ ((row >> 1) & 3)) << 4)  in shared
// memory, which spreads the eight rows of a ldmatrix phase over all banks.  The sums are staged in the row-major
// layout of the row-wise pass (over the Qt tile, which is dead by then) and leave as whole 256-byte rows.
__device__ __forceinline__ uint32_t vt_off(int row, int tok) {
  return (uint32_t)row * 64u + (uint32_t)(((tok >> 3) ^ ((row >> 1) & 3)) << 4) + (uint32_t)(tok & 7) * 2u;
}

__global__ void __launch_bounds__(FIX_THREADS) kda_fixup_tiles_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ tiles,
                                                                      long long oloc_tile_offset, long long ldo,
                                                                      const float* __restrict__ S_in, const long long* __restrict__ t0s,
                                                                      const long long* __restrict__ t1s, const int* __restrict__ need_map,
                                                                      int n_seg, int H, long long T, int split) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slice = blockIdx.x % split;
  const int h = (blockIdx.x / split) % H;
  const int seg = blockIdx.x / (split * H);
  if (seg >= n_seg || !need_map[seg]) return;
  const long long t0 = max(0LL, t0s[seg]), t1 = min(T, t1s[seg]);
  if (t1 <= t0) return;
  const int ntiles = (int)((t1 - t0 + 31) / 32);
  if (slice >= ntiles) return;
  const __nv_bfloat16* qt_tiles = tiles + (seg_tile0(t0s, t1s, T, seg) * H + h) * (D * C);

  // entering state -> bf16 [v][k'] tile (row = value index: the B operand with k' contiguous)
  const float* S = S_in + ((size_t)seg * H + h) * STATE_ELEMS;
  for (int idx = tid; idx < D * D / 4; idx += FIX_THREADS) {
    const int row = idx >> 5, c4 = (idx & 31) * 4;
    const float4 f = *reinterpret_cast<const float4*>(S + row * D + c4);
    *reinterpret_cast<uint2*>(smem + tile128_off(row, c4)) = make_uint2(pack_bf16(f.x, f.y), pack_bf16(f.z, f.w));
  }
  const uint32_t s_tile = smem_u32(smem);
  const int g = lane >> 2, t = lane & 3;
  const int frag_row = 8 * (lane >> 4) + (lane & 7);
  const int frag_chunk = (lane >> 3) & 1;

  auto issue = [&](int tile, int buf) {
    const __nv_bfloat16* src = qt_tiles + (size_t)tile * H * (D * C);
    const uint32_t dst = smem_u32(smem + 32768 + buf * 16384);
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const int idx = tid + FIX_THREADS * j, row = idx >> 2, piece = idx & 3;
      const uint32_t soff = row * 64 + ((piece ^ ((row >> 1) & 3)) << 4);
      cp_async16(dst + soff, src + idx * 8, 16);
      cp_async16(dst + 8192 + soff, src + oloc_tile_offset + idx * 8, 16);
    }
  };
  issue(slice, 0);
  cp_async_commit();
  int buf = 0;
  for (int tile = slice; tile < ntiles; tile += split, buf ^= 1) {
    if (tile + split < ntiles) issue(tile + split, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    uint8_t* q_buf = smem + 32768 + buf * 16384;
    const uint32_t q_tile = smem_u32(q_buf);
    const uint8_t* o_tile = q_buf + 8192;
    float acc[2][2][4];
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
      for (int b = 0; b < 2; b++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[a][b][c] = 0.0f;
    // A fragment (16 tokens x 16 k') from the [k'][token] tile: matrix m of the ldmatrix covers tokens 8 (m & 1) ..,
    // k' 8 (m >> 1) ..; lanes 8 m .. 8 m + 7 give the addresses of its eight k' rows
    const int a_tok = 8 * ((lane >> 3) & 1), a_k = 8 * (lane >> 4) + (lane & 7);
#pragma unroll
    for (int kt = 0; kt < 8; kt++) {
      uint32_t b[4];
      ldmatrix_x4(b, s_tile + tile128_off(16 * warp + frag_row, (2 * kt + frag_chunk) * 8));
#pragma unroll
      for (int mt = 0; mt < 2; mt++) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, q_tile + vt_off(16 * kt + a_k, 16 * mt + a_tok));
        mma_bf16(acc[mt][0], a, b[0], b[1]);
        mma_bf16(acc[mt][1], a, b[2], b[3]);
      }
    }
    // + o_loc (row = value index, token along the row)
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const int tok = 16 * mt + g + 8 * half;
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
          const int vv = 16 * warp + 8 * nt + 2 * t;
          acc[mt][nt][2 * half] += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(o_tile + vt_off(vv, tok)));
          acc[mt][nt][2 * half + 1] += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(o_tile + vt_off(vv + 1, tok)));
        }
      }
    __syncthreads();                               // every warp is done with the Qt tile: the sums take its place
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const int row = 16 * mt + g + 8 * half;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
          *reinterpret_cast<uint32_t*>(q_buf + tile128_off(row, 16 * warp + 8 * nt + 2 * t)) =
              pack_bf16(acc[mt][nt][2 * half], acc[mt][nt][2 * half + 1]);
      }
    __syncthreads();
    const long long tok0 = t0 + (long long)tile * 32;
    const int nvalid = (int)min(32LL, t1 - tok0);
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const int idx = tid + FIX_THREADS * j, row = idx >> 4, ch = idx & 15;
      if (row < nvalid)
        *reinterpret_cast<uint4*>(out + (tok0 + row) * ldo + (long long)h * D + ch * 8) =
            *reinterpret_cast<const uint4*>(q_buf + row * 256 + ((ch ^ (row & 7)) << 4));
    }
    __syncthreads();
  }
}

cudaError_t launch_fixup_tiles(__nv_bfloat16* out, const __nv_bfloat16* tiles, long long oloc_tile_offset, long long ldo,
                               const float* S_in, const long long* t0, const long long* t1, const int* need_map, int n_seg,
                               int H, long long T, cudaStream_t stream) {
  static int attr_dev_mask = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(attr_dev_mask & (1 << (dev & 31)))) {
    cudaError_t e = cudaFuncSetAttribute(kda_fixup_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FIX_SMEM);
    if (e != cudaSuccess) return e;
    attr_dev_mask |= 1 << (dev & 31);
  }
  int split = (16 * 148 + n_seg * H - 1) / (n_seg * H);   // about sixteen CTAs per SM: short waves, 5 % faster than four
  if (split < 1) split = 1;
  if (split > 64) split = 64;
  kda_fixup_tiles_kernel<<<(unsigned)(n_seg * H * split), FIX_THREADS, FIX_SMEM, stream>>>(out, tiles, oloc_tile_offset, ldo, S_in, t0, t1,
                                                                                           need_map, n_seg, H, T, split);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ state rows
__global__ void __launch_bounds__(256) kda_rows_copy_kernel(void* __restrict__ dst, long long dst_row_stride, int dst_is_bf16,
                                                            const float* __restrict__ src, long long src_row_stride,
                                                            const int* __restrict__ idx, int H) {
  const int row = blockIdx.x / H, h = blockIdx.x % H;
  const long long srow = idx ? idx[row] : row;
  if (srow < 0) return;
  const float4* s = reinterpret_cast<const float4*>(src + srow * src_row_stride + (size_t)h * STATE_ELEMS);
  if (dst_is_bf16) {
    uint2* d = reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(dst) + row * dst_row_stride + (size_t)h * STATE_ELEMS);
#pragma unroll 4
    for (int i = threadIdx.x; i < STATE_ELEMS / 4; i += 256) {
      const float4 f = s[i];
      d[i] = make_uint2(pack_bf16(f.x, f.y), pack_bf16(f.z, f.w));
    }
  } else {
    float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + row * dst_row_stride + (size_t)h * STATE_ELEMS);
#pragma unroll 4
    for (int i = threadIdx.x; i < STATE_ELEMS / 4; i += 256) d[i] = s[i];
  }
}

cudaError_t launch_rows_copy(void* dst, long long dst_row_stride, int dst_is_bf16, const float* src, long long src_row_stride,
                             const int* idx, int n_rows, int H, cudaStream_t stream) {
  kda_rows_copy_kernel<<<(unsigned)(n_rows * H), 256, 0, stream>>>(dst, dst_row_stride, dst_is_bf16, src, src_row_stride, idx, H);
  return cudaGetLastError();
}

}  // namespace kda
