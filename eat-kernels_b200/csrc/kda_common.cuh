// Shared device-side definitions of the KDA prefill kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kda {

constexpr int D = 128;          // head dim (K = V)
constexpr int C = 32;           // tokens per chunk
constexpr int HALF = 16;        // sub-chunk: reference exponent taken after token HALF-1
constexpr int STATE_ELEMS = D * D;
constexpr float LOG2E = 1.4426950408889634f;

// The task count word the planner leaves for the chunk kernels: count in the low bits, plus this bit when cu_seqlens was
// rejected and the launch has to zero-fill the output rows (one word, so that a CTA without a task exits after a
// single load: capacity-sized grids are mostly such CTAs).
constexpr int NT_ZERO_FILL = 1 << 30;

// Task flags
constexpr uint32_t TF_INIT_ZERO = 1u;      // start from S = 0
constexpr uint32_t TF_INIT_IDENTITY = 2u;  // start from S = I (transition chain)
constexpr uint32_t TF_V_ZERO = 4u;         // treat v as 0 (transition chain)
constexpr uint32_t TF_OUT_AUX = 8u;        // write output rows to the auxiliary tensor (Qt)
constexpr uint32_t TF_NO_OUT = 16u;        // do not write output rows
constexpr uint32_t TF_DUAL = 64u;          // tcgen05 kernel only: run chain L (this task's own flags, real v -> out, dst) AND
                                           // chain Tr (S = I, v = 0 -> out_aux, dst2) over one operand preparation
constexpr uint32_t TF_DST_VF = 32u;        // store the final state value-first whatever the launch's state layout
                                           // (transition maps: the scan applies them as  E <- E P)

// One unit of work of the fused chunk kernel: a run of tokens of one sequence (all heads).
struct __align__(16) Task {
  long long t0;        // first token row
  int len;             // tokens
  uint32_t flags;
  const float* src;    // initial state of head 0 (heads 16384 floats apart); unused with TF_INIT_*
  float* dst;          // final state of head 0, or nullptr
  void* ck;            // first checkpoint row of this run (head 0), or nullptr; TF_DUAL tasks that write output: the
                       // task's first Qt tile (head 0) in the tile-major scratch (see role_tmem_dual)
  float* dst2;         // TF_DUAL: final state of the transition chain (head 0, always value-first); else unused
};

struct ChunkParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const void* g;
  const void* beta;
  __nv_bfloat16* out;
  __nv_bfloat16* out_aux;
  long long oloc_tile_offset;  // dual-chain tasks with output: elements from a task's Qt tiles to its o_loc tiles
  long long ldq, ldk, ldv, ldg, ldbeta, ldo;
  const float* A_log;
  const float* dt_bias;
  float scale, lower_bound;
  int frontend;        // 0 raw, 1 plain
  int key_first;       // state layout
  int H;
  int ck_is_bf16;
  int ck_every_chunks; // checkpoint interval in chunks (0 = off)
  long long ck_row_stride;   // elements between consecutive checkpoint rows (H * 16384)
  const Task* tasks;
  const int* n_tasks;  // device: number of valid tasks
  int* status;         // device int[4]
  long long T;         // token rows (for the zero-fill of a rejected layout)
  unsigned long long wait_limit_ns;   // bound of every in-kernel wait (0 = the built-in default)
  int debug_flags;     // DBG_* below; 0 in every product launch
  unsigned long long* prof;           // cycle counters of profiling builds (KDA_PROF), else unused
};

// Diagnostic switches of the tcgen05 kernel (set only through kda_debug_configure).
constexpr int DBG_STALL_V_STREAM = 1;  // the v tiles never count as arrived: their waiters run into the bound
// bits 8-11: k + 1 makes the device planner take candidate k of its piece lengths (a tuning aid for the cost model)
constexpr int DBG_FORCE_CAND_SHIFT = 8, DBG_FORCE_CAND_MASK = 0xf00;

// ----------------------------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void stmatrix_x4_trans(uint32_t addr, const uint32_t (&r)[4]) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1,%2,%3,%4};\n"
               :: "r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}

// D (fp32, 16x8) += A (bf16, 16x16 row) * B (bf16, 16x8 col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// D (fp32, 16x8) += A (tf32, 16x8 row) * B (tf32, 8x8 col); operands are fp32 bit patterns (low mantissa bits ignored)
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N) : "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;\n" :: "r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float bf16_lo(uint32_t x) { return __uint_as_float(x << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t x) { return __uint_as_float(x & 0xffff0000u); }

// packed fp32 pairs (one instruction for two lanes of arithmetic on sm_100)
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2,%3};\n mov.b64 rb, {%4,%5};\n mul.rn.f32x2 rd, ra, rb;\n mov.b64 {%0,%1}, rd;\n}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcpf(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// sigmoid with relative accuracy for small results (needed by slow gates: sigmoid(-9) must keep its digits)
__device__ __forceinline__ float sigmoidf_rel(float x) { return rcpf(1.0f + ex2f(-x * LOG2E)); }

// Byte offset of element (row, col) of a [rows][128] bf16 tile with 256-byte rows, 16-byte chunks XOR-swizzled by
// row so that the eight rows of an ldmatrix phase fall into distinct banks.
__device__ __forceinline__ uint32_t tile128_off(int row, int col) {
  return static_cast<uint32_t>(row * 256 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1)));
}
// Same for a [32][32] bf16 tile with 64-byte rows (4 chunks per row).
__device__ __forceinline__ uint32_t tile32_off(int row, int col) {
  return static_cast<uint32_t>(row * 64 + ((((col >> 3) ^ ((row >> 1) & 3)) << 4) | ((col & 7) << 1)));
}

}  // namespace kda
