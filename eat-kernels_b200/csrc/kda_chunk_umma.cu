// Fused KDA chunk kernel on the 5th-generation tensor core (tcgen05 + tensor memory), sm_100a.
//
// One CTA walks the 32-token chunks of one (token run, head) task.  The fp32 state St [V=128][K=128] (value-first) never
// leaves tensor memory between chunks, and the whole per-chunk chain is tensor-core work issued by one elected lane:
//
//   MMA1  [W | O] = St [kd ; qd]^T          tf32: A = St read straight from its accumulator columns, N = 64, K = 128
//   MMA2  U  = v^T Tbh^T - W Tb^T           bf16 (A = v tile, MN-major) then tf32 (A = W columns, B negated), N = 32, K = 32
//   MMA3  St += U kr ,  O += U M^T          tf32: A = U columns; kr MN-major (N = 128), M K-major (N = 32)
//
// with kd = k 2^G, qd = scale q 2^G, kr = k 2^(G31-G), Tb = (I + diag(beta) tril(kd' ki'^T,-1))^-1 diag(beta),
// M = tril(qd' ki'^T) (G = inclusive cumulative log2-decay of the chunk; primed operands are taken relative to the
// exponent after token 15 so that every exponent is bounded by the decay of 16 tokens).  This is the chunked form of
// kda/b200/reference.py:30-37.  No accumulator makes a round trip through registers on the chain; the only register
// pass is the per-chunk decay St <- St diag(2^G31), done by the eight tensor-memory warps between MMA1 and MMA3, off
// the MMA warp's issue path.  Because tf32 operands keep 10 mantissa bits, the state enters the products more accurately
// than a bf16 copy would.
//
// Warp roles (28 warps):
//    0      MMA issuer (+ tensor-memory allocation); the whole warp runs the issue loop on warp-uniform values
//    1-2    triangular inverse, alternating chunks
//    3      loader: one lane polls three TMA copy streams (g / q,k / v); v goes straight into the consumer stage
//    4-11   tensor-memory warps: state load, per-chunk decay, checkpoints, final store, and O -> bf16 -> global; each
//           warp serves half of the columns of one lane quarter
//    12-27  operand preparation in two groups of eight warps that alternate chunks: gate + cumsum, L2 norm, decayed
//           operand tiles, intra-chunk products on mma.sync
// Roles hand off through mbarriers; every wait is bounded (see kda_umma.cuh): on a timeout the CTA keeps its control
// flow, waits (bounded again) for its copies and tensor-core work in flight, frees tensor memory and reports an error
// code in status[2].
//
// Measured alternative, not kept: the intra-chunk products as one bf16 tcgen05.mma over interleaved q / k tiles with
// the two results pulled out of tensor memory by the inverse warps.  It halves the work of the preparation warps, but
// the tensor-core round trip (issue, commit, barrier, tensor-memory load) and the extraction sit on the chain
// tiles -> products -> inverse -> MMA2, which with two operand stages is what sets the per-chunk time: 3-13 % slower.
#include "kda_common.cuh"
#include "kda_plan.cuh"
#include "kda_tma.cuh"
#include "kda_umma.cuh"

namespace kda {
using namespace umma;

namespace u {

constexpr int WARPS = 28;
constexpr int THREADS = WARPS * 32;
constexpr int W_MMA = 0, W_INV0 = 1, W_LOAD = 3, W_SCALE0 = 4, W_PREP0 = 12;
constexpr int PREP_GROUPS = 2;                 // group g prepares the chunks c with c % 2 == g, in stage g
constexpr int PREP_WARPS = 8, PREP_THREADS = 256;   // per group

// ---- shared memory map (bytes); operand tiles are 1024-byte aligned
constexpr int CS_KDQD = 0, CS_KR = 32768, CS_V = 49152, CS_TB = 57344, CS_M = 61440, CS_STAGE = 65536;
constexpr int OFF_CONS = 0;                                   // 2 stages
constexpr int RAW_G = 0, RAW_Q = 16384, RAW_K = 24576, RAW_STAGE = 32768;
constexpr int OFF_RAW = OFF_CONS + 2 * CS_STAGE;              // 2 stages
constexpr int OFF_KIS = OFF_RAW + 2 * RAW_STAGE;              // 2 x 8192 (one per prep group)
constexpr int OFF_TBH = OFF_KIS + 2 * 8192;                   // 2 x 2048 (bf16, 64-byte swizzle)
constexpr int OFF_L = OFF_TBH + 4096;                         // 2 x 4096 fp32 [32][32]
constexpr int OFF_DEC = OFF_L + 8192;                         // 4 x 512 (a slot is rewritten four chunks later)
constexpr int OFF_FR = OFF_DEC + 2048;                        // per prep group: (free), 2^r, first-half sum then 2^(G31-r) : 2 x 3 x 512
constexpr int OFF_BETA = OFF_FR + 2 * 1536;                   // raw-stage beta: 2 x 128
constexpr int OFF_LBETA = OFF_BETA + 256;                     // beta next to L: 2 x 128
constexpr int OFF_BAR = OFF_LBETA + 256;                      // mbarriers
constexpr int NUM_BARS = 42;
constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;              // +0 tmem slot, +8 abort code, +12 range flag, +16 wait limit (ns)
constexpr int SMEM_BYTES = OFF_MISC + 64;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");

// mbarrier indices
constexpr int B_G_FULL = 0, B_G_EMPTY = 2, B_CONS_EMPTY = 4, B_P1_FULL = 6, B_INV_FULL = 8, B_L_FULL = 10,
              B_L_EMPTY = 12, B_O_FULL = 14, B_O_EMPTY = 16, B_MMA1_DONE = 18, B_S_READY = 19, B_DRAIN = 20, B_V_EMPTY = 21,
              B_QK_FULL = 23, B_QK_EMPTY = 25, B_V_FULL = 27, B_KDQD_EMPTY = 29,
              B_MMA1_DONE_T = 31, B_S_READY_T = 32,   // second chain of a dual-chain task
              B_TOT = 34;                             // 2 groups x 4 warp pairs: first-half sums of step A

// tensor-memory columns
constexpr uint32_t TM_COLS = 512, TM_S = 0, TM_WO = 128, TM_U = 256;
constexpr uint32_t TD_S0 = 0, TD_S1 = 128, TD_WO0 = 256, TD_WO1 = 320, TD_U0 = 384, TD_U1 = 448;   // dual-chain tasks

// error codes written to status[2] when a bounded wait gives up (which role, which barrier)
constexpr int E_LOAD = 0x40, E_PREP = 0x80, E_INV = 0xc0, E_MMA = 0x100, E_SCALE = 0x140, E_EPI = 0x180, E_DRAIN = 0x1c0;

#ifdef KDA_PROF
#define PROF_STAMP(role, slot) do { if ((threadIdx.x & 31) == 0 && blockIdx.x == 0 && x.prof != nullptr) { const long long _t = clock64(); atomicAdd(x.prof + (role) * 128 + 64 + (slot), (unsigned long long)(_t - prof_last)); prof_last = _t; } } while (0)
#define PROF_BEGIN long long prof_last = clock64()
#else
#define PROF_STAMP(role, slot) do { } while (0)
#define PROF_BEGIN do { } while (0)
#endif

// Byte offset of element (row, col) of a raw / decayed bf16 [32][128] tile as the copy engine lays it out with the
// 128-byte swizzle: two halves of 64 channels, each 32 rows of 128 bytes, 16-byte chunks XOR-ed with (row % 8).
// ldmatrix phases (8 rows, one chunk) are bank-conflict free in this layout.
__device__ __forceinline__ uint32_t rawtile_off(int row, int col) {
  return (uint32_t)((col >> 6) * 4096 + row * 128 + (((((col & 63) >> 3) ^ (row & 7))) << 4) + ((col & 7) << 1));
}

#ifndef KDA_SLEEP_NS
#define KDA_SLEEP_NS 32
#endif
constexpr unsigned kSleepNs = KDA_SLEEP_NS;   // back-off of waiting warps (not of the MMA issuer)

struct Ctx {
  uint8_t* smem;
  uint32_t bars;              // shared address of barrier 0
  volatile int* abort_flag;
  int h, len, nchunks;
  long long t0;
  __device__ __forceinline__ uint32_t bar(int i) const { return bars + 8u * (uint32_t)i; }
#ifdef KDA_PROF
  unsigned long long* prof;   // [role 0..7][wait on barrier 0..63 | 64 + stamp slot | 126 = total, 127 = warps] cycle
                              // counters of CTA 0 (profiling builds only; a buffer of its own, see kda_debug_configure)
  __device__ __forceinline__ void wait(int i, uint32_t parity, int code, unsigned sleep_ns = kSleepNs) const {
    const long long t = clock64();
    mbar_wait(bar(i), parity, abort_flag, code + i, sleep_ns);
    if ((threadIdx.x & 31) == 0 && blockIdx.x == 0 && prof != nullptr)
      atomicAdd(prof + ((code >> 6) * 128 + i), (unsigned long long)(clock64() - t));
  }
#else
  __device__ __forceinline__ void wait(int i, uint32_t parity, int code, unsigned sleep_ns = kSleepNs) const {
    mbar_wait(bar(i), parity, abort_flag, code + i, sleep_ns);
  }
#endif
};

// ------------------------------------------------------------------------------------------------ loader warp
// One elected lane drives the copy engine: per chunk it arms the stage's mbarrier with the byte count and issues the
// tile copies (g, q, k into the raw stage, v straight into the MMA2 operand slot of the consumer stage, whose
// MN-major 128-byte-swizzled layout is exactly what the engine writes).
// Rare paths of the loader, out of line: its polling loop sits on the refill latency of every tile, and anything that
// adds live state or code to it costs measurable time per chunk.
__device__ __noinline__ bool loader_idle_expired(unsigned long long idle_ns, volatile int* abort_flag) {
  if (idle_ns <= wait_limit_of(abort_flag)) return false;
  atomicCAS(const_cast<int*>(abort_flag), 0, E_LOAD);
  return true;
}
// Before the CTA may leave, every copy the loader issued has landed (on the normal path the consumers saw to that
// long ago and these waits return at once; after a give-up they keep the copy engine from writing into a dead CTA).
// A stage's full barrier is not re-armed after its last copy, so the parity of that last phase is still testable.
__device__ __noinline__ void loader_drain(uint32_t bars, volatile int* abort_flag, int cg, int cq, int cv) {
#pragma unroll 1
  for (int st = 0; st < 3; st++) {
    const int issued = st == 0 ? cg : (st == 1 ? cq : cv);
    const int fb = st == 0 ? B_G_FULL : (st == 1 ? B_QK_FULL : B_V_FULL);
    for (int c = max(0, issued - 2); c < issued; c++)
      if (!mbar_wait_drain(bars + 8u * (uint32_t)(fb + (c & 1)), (uint32_t)((c >> 1) & 1), abort_flag))
        atomicCAS(const_cast<int*>(abort_flag), 0, E_DRAIN + fb);
  }
}

template <int FE>
__device__ void role_loader(const ChunkParams& p, const TmaMaps& m, const Ctx& x, int lane) {
  // Three independent copy streams (g; q and k; v), each with its own full / empty barrier pair per stage: the gate
  // tile is free after step B of the chunk two back, q / k after step C, v only once MMA2 has read it.  ONE lane
  // serves all three by polling the empty barriers without blocking: a blocking wait of one stream (or of a second
  // lane of this warp, which shares the warp's single scheduling slot) would delay the refill of the others by its
  // suspend time, and the refill latency of q / k sits on the chain  copy -> step B -> step C -> inverse -> MMA2.
  if (lane != 0) return;
  const int n = x.nchunks;
  int cg = 0, cq = 0, cv = 0;                 // next chunk of each stream
  unsigned idle = 0;
  unsigned long long t_idle = 0;
#pragma unroll 1
  while (cg < n || cq < n || cv < n) {
    bool progressed = false;
    if (cq < n) {
      const int s = cq & 1;
      if (mbar_test_wait(x.bar(B_QK_EMPTY + s), (uint32_t)(((cq >> 1) & 1) ^ 1))) {
        uint8_t* raw = x.smem + OFF_RAW + s * RAW_STAGE;
        const uint32_t qraw = smem_u32(raw + RAW_Q), kraw = smem_u32(raw + RAW_K);
        const int tok0 = (int)(x.t0 + (long long)cq * C);
        tma::mbar_arrive_expect_tx(x.bar(B_QK_FULL + s), 2u * 8192u);
        tma::load_3d(qraw, &m.q, 0, x.h, tok0, x.bar(B_QK_FULL + s));
        tma::load_3d(qraw + 4096, &m.q, 64, x.h, tok0, x.bar(B_QK_FULL + s));
        tma::load_3d(kraw, &m.k, 0, x.h, tok0, x.bar(B_QK_FULL + s));
        tma::load_3d(kraw + 4096, &m.k, 64, x.h, tok0, x.bar(B_QK_FULL + s));
        cq++;
        progressed = true;
      }
    }
    if (cg < n) {
      const int s = cg & 1;
      if (mbar_test_wait(x.bar(B_G_EMPTY + s), (uint32_t)(((cg >> 1) & 1) ^ 1))) {
        uint8_t* raw = x.smem + OFF_RAW + s * RAW_STAGE;
        const int tok0 = (int)(x.t0 + (long long)cg * C);
        tma::mbar_arrive_expect_tx(x.bar(B_G_FULL + s), FE == 1 ? 16384u : 8192u);
        tma::load_3d(smem_u32(raw + RAW_G), &m.g, 0, x.h, tok0, x.bar(B_G_FULL + s));
        cg++;
        progressed = true;
      }
    }
    if (cv < n) {
      const int s = cv & 1;
      if (mbar_test_wait(x.bar(B_V_EMPTY + s), (uint32_t)(((cv >> 1) & 1) ^ 1))) {
        const uint32_t vdst = smem_u32(x.smem + OFF_CONS + s * CS_STAGE + CS_V);
        const int tok0 = (int)(x.t0 + (long long)cv * C);
        tma::mbar_arrive_expect_tx(x.bar(B_V_FULL + s), 8192u);
        tma::load_3d(vdst, &m.v, 0, x.h, tok0, x.bar(B_V_FULL + s));
        tma::load_3d(vdst + 4096, &m.v, 64, x.h, tok0, x.bar(B_V_FULL + s));
        cv++;
        progressed = true;
      }
    }
    if (progressed) {
      idle = 0;
      t_idle = 0;
    } else {
      // nothing to refill yet: back off briefly; give up like every other wait of the kernel does
      __nanosleep(32);
      if (*x.abort_flag != 0) break;
      if ((++idle & 1023u) == 0) {
        const unsigned long long now = global_timer_ns();
        if (t_idle == 0) t_idle = now;
        else if (loader_idle_expired(now - t_idle, x.abort_flag)) break;
      }
    }
  }
  loader_drain(x.bars, x.abort_flag, cg, cq, (p.debug_flags & DBG_STALL_V_STREAM) ? 0 : cv);
}

template <int FE>
__device__ __forceinline__ float load_beta(const ChunkParams& p, const Ctx& x, int c, int row) {
  const int nvalid = min(C, x.len - c * C);
  if (row >= nvalid) return 0.0f;
  const long long tok = x.t0 + (long long)c * C + row;
  if (FE == 1) return reinterpret_cast<const float*>(p.beta)[tok * p.ldbeta + x.h];
  return sigmoidf_rel(__bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.beta)[tok * p.ldbeta + x.h]));
}

// ------------------------------------------------------------------------------------------------ prep warps
template <int FE>
__device__ void role_prep(const ChunkParams& p, const Ctx& x, int grp, int ptid) {
  const int pw = ptid >> 5, lane = ptid & 31;
  const int ch = ptid & 127, half = ptid >> 7;
  const int s = grp;                                   // the group's raw and consumer stage
  const int bar_id = 1 + grp;
  float eA = 0.0f, dtb = 0.0f;
  if (FE == 0) {
    eA = __expf(p.A_log[x.h]);
    dtb = p.dt_bias[x.h * D + ch];
  }
  float* fr = reinterpret_cast<float*>(x.smem + OFF_FR) + grp * 3 * D;
  float* fer = fr + D;
  float* tot = fr + 2 * D;
  uint8_t* raw = x.smem + OFF_RAW + s * RAW_STAGE;
  uint8_t* cons = x.smem + OFF_CONS + s * CS_STAGE;
  uint8_t* kis_tile = x.smem + OFF_KIS + grp * 8192;
  float* Gsm = reinterpret_cast<float*>(raw + RAW_G);
  float* beta_s = reinterpret_cast<float*>(x.smem + OFF_BETA) + s * 32;
  volatile int* range_flag = reinterpret_cast<volatile int*>(x.smem + OFF_MISC + 12);
  float beta_next = (ptid < C && grp < x.nchunks) ? load_beta<FE>(p, x, grp, ptid) : 0.0f;   // one own chunk ahead
#pragma unroll 1
  for (int c = grp; c < x.nchunks; c += PREP_GROUPS) {
    const uint32_t par = (uint32_t)((c >> 1) & 1);
    const int nvalid = min(C, x.len - c * C);
    float* dec = reinterpret_cast<float*>(x.smem + OFF_DEC) + (c & 3) * D;
    x.wait(B_G_FULL + s, par, E_PREP);
    PROF_BEGIN;

    // ---- A: gate activation + inclusive cumulative log2-decay; two threads per channel, 16 tokens each.
    // Touches only prep-private scratch (the decay slot c & 3 was last read four chunks ago), so it runs while the
    // tensor core still works on older chunks.
    {
      float a[16];
      if (FE == 1) {
        const float* g = reinterpret_cast<const float*>(raw + RAW_G);
#pragma unroll
        for (int i = 0; i < 16; i++) a[i] = g[(16 * half + i) * D + ch];
      } else {
        // log2-decay = lower_bound log2(e) sigmoid(x), x = exp(A_log) (g + dt_bias); sigmoid(x) = 1 / (1 + 2^(-x log2 e))
        // with the exponent argument formed by one fused multiply-add per element
        const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(raw + RAW_G);
        const float m1 = -LOG2E * eA, m0 = m1 * dtb;
#pragma unroll
        for (int i = 0; i < 16; i++) a[i] = rcpf(1.0f + ex2f(fmaf(__bfloat162float(g[(16 * half + i) * D + ch]), m1, m0)));
      }
      if (nvalid < C) {                       // rows of the next sequence (last chunk only): no decay
#pragma unroll
        for (int i = 0; i < 16; i++)
          if (16 * half + i >= nvalid) a[i] = 0.0f;
      }
      // inclusive cumulative sum in log2 units, the unit conversion fused into the additions
      const float unit = (FE == 1) ? LOG2E : p.lower_bound * LOG2E;
      a[0] *= unit;
#pragma unroll
      for (int i = 1; i < 16; i++) a[i] = fmaf(a[i], unit, a[i - 1]);
      if (FE == 1) {
        // fp32 gates are replaced in place by the thread that read them, so only the first-half sums cross threads:
        // warp pw hands the sums of its 32 channels to warp pw + 4 through a barrier of their own.
        if (half == 0) {
          tot[ch] = a[15];
          __syncwarp();
          if (lane == 0) mbar_arrive(x.bar(B_TOT + 4 * grp + pw));
        } else {
          x.wait(B_TOT + 4 * grp + (pw - 4), par, E_PREP);
        }
        PROF_STAMP(2, 10);
        PROF_STAMP(2, 11);
      } else {
        if (half == 0) tot[ch] = a[15];
        PROF_STAMP(2, 10);
        named_bar_sync(bar_id, PREP_THREADS);   // all raw g values are in registers: the exponents may now overwrite the tile
        PROF_STAMP(2, 11);
      }
      // What step B needs is the exponent relative to r = G after token 15, clamped to the representable range:
      // tokens 0-15 have G - r = own sum - r >= 0, tokens 16-31 have G - r = their own partial sum <= 0.
      if (half == 1) {
        const float r = tot[ch];
        // Range of the primed operands: the largest exponents belong to token 0 (at most -r) and token 31 (a[15], the
        // second half's own sum).  Beyond 2^126 they are clamped and the intra-chunk products of this chunk are no
        // longer exact: report it.  (Checked here, by the threads that hold both numbers anyway, and reported by one
        // lane per warp: these warps set the pace of the kernel, and a separate test in the first half of step A cost
        // 2.7 % of it.)
        if (__any_sync(0xffffffffu, fminf(r, a[15]) < -126.0f) && lane == 0) *range_flag = 1;
        fer[ch] = ex2f(r);
        dec[ch] = ex2f(a[15] + r);
        tot[ch] = ex2f(a[15]);          // 2^(G31 - r), read back below as the kr factor
#pragma unroll
        for (int i = 0; i < 16; i++) a[i] = fmaxf(a[i], -126.0f);
      } else {
        const float r = a[15];
#pragma unroll
        for (int i = 0; i < 16; i++) a[i] = fminf(a[i] - r, 126.0f);
      }
#pragma unroll
      for (int i = 0; i < 16; i++) Gsm[(16 * half + i) * D + ch] = a[i];
    }
    PROF_STAMP(2, 12);
    named_bar_sync(bar_id, PREP_THREADS);
    PROF_STAMP(2, 26);
    // Every warp of the group has left the previous chunk (step C reads beta_s), so beta may be replaced only now; step
    // C of this chunk reads it after the next barrier.
    if (ptid < C) {
      beta_s[ptid] = beta_next;
      if (c + PREP_GROUPS < x.nchunks) beta_next = load_beta<FE>(p, x, c + PREP_GROUPS, ptid);
    }

    // ---- B: L2 norm and decayed operand tiles; a warp owns 4 tokens, a lane 4 channels.  [kd ; qd] is written as
    // soon as MMA1 of the chunk two back has read the stage; kr waits in registers until MMA3 has released the rest.
    x.wait(B_QK_FULL + s, par, E_PREP);
    x.wait(B_KDQD_EMPTY + s, par ^ 1, E_PREP);
    PROF_STAMP(2, 14);
    float krr[4][4];
    {
      const float4 er4 = *reinterpret_cast<const float4*>(fer + 4 * lane);
      const float4 elr4 = *reinterpret_cast<const float4*>(tot + 4 * lane);
      const float er[4] = {er4.x, er4.y, er4.z, er4.w};
      const float elr[4] = {elr4.x, elr4.y, elr4.z, elr4.w};
#pragma unroll
      for (int tt = 0; tt < 4; tt++) {
        const int tok = 4 * pw + tt;
        const uint32_t off = rawtile_off(tok, 4 * lane);
        uint2 q2 = *reinterpret_cast<const uint2*>(raw + RAW_Q + off);
        uint2 k2 = *reinterpret_cast<const uint2*>(raw + RAW_K + off);
        if (nvalid < C && tok >= nvalid) { q2 = make_uint2(0u, 0u); k2 = make_uint2(0u, 0u); }   // rows of the next sequence
        const float qf[4] = {bf16_lo(q2.x), bf16_hi(q2.x), bf16_lo(q2.y), bf16_hi(q2.y)};
        const float kf[4] = {bf16_lo(k2.x), bf16_hi(k2.x), bf16_lo(k2.y), bf16_hi(k2.y)};
        float qinv = p.scale, kinv = 1.0f;
        if (FE == 0) {
          float sq = qf[0] * qf[0] + qf[1] * qf[1] + qf[2] * qf[2] + qf[3] * qf[3];
          float sk = kf[0] * kf[0] + kf[1] * kf[1] + kf[2] * kf[2] + kf[3] * kf[3];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
            sk += __shfl_xor_sync(0xffffffffu, sk, o);
          }
          qinv = p.scale * rsqrtf(fmaxf(sq, 1e-12f));   // x / max(||x||, 1e-6)
          kinv = rsqrtf(fmaxf(sk, 1e-12f));
        }
        const float4 G4 = *reinterpret_cast<const float4*>(Gsm + tok * D + 4 * lane);
        const float Gv[4] = {G4.x, G4.y, G4.z, G4.w};
        float kds[4], qds[4], kis[4], kdt[4], qdt[4];
#pragma unroll
        for (int j = 0; j < 4; j += 2) {               // channel pairs, packed fp32x2 arithmetic
          const float e0 = Gv[j], e1 = Gv[j + 1];
          const float2 E = make_float2(ex2f(e0), ex2f(e1)), Ei = make_float2(ex2f(-e0), ex2f(-e1));
          float2 kn = make_float2(kf[j], kf[j + 1]);
          if (FE == 0) kn = mul2(kn, make_float2(kinv, kinv));
          const float2 qn = mul2(make_float2(qf[j], qf[j + 1]), make_float2(qinv, qinv));
          const float2 kd2 = mul2(kn, E), qd2 = mul2(qn, E), ki2 = mul2(kn, Ei);
          const float2 er2 = make_float2(er[j], er[j + 1]);
          const float2 kt2 = mul2(kd2, er2), qt2 = mul2(qd2, er2), kr2 = mul2(ki2, make_float2(elr[j], elr[j + 1]));
          kds[j] = kd2.x; kds[j + 1] = kd2.y; qds[j] = qd2.x; qds[j + 1] = qd2.y; kis[j] = ki2.x; kis[j + 1] = ki2.y;
          kdt[j] = kt2.x; kdt[j + 1] = kt2.y; qdt[j] = qt2.x; qdt[j + 1] = qt2.y; krr[tt][j] = kr2.x; krr[tt][j + 1] = kr2.y;
        }
        // in place: the decayed bf16 tiles of the intra-chunk products replace the raw q / k tiles
        *reinterpret_cast<uint2*>(raw + RAW_K + off) = make_uint2(pack_bf16(kds[0], kds[1]), pack_bf16(kds[2], kds[3]));
        *reinterpret_cast<uint2*>(raw + RAW_Q + off) = make_uint2(pack_bf16(qds[0], qds[1]), pack_bf16(qds[2], qds[3]));
        *reinterpret_cast<uint2*>(kis_tile + off) = make_uint2(pack_bf16(kis[0], kis[1]), pack_bf16(kis[2], kis[3]));
        // tf32 operands of the state products: [kd ; qd] K-major (row = token, 32 + token), kr MN-major
        *reinterpret_cast<float4*>(cons + CS_KDQD + kmajor_f32_off(tok, 4 * lane, 8192)) = make_float4(kdt[0], kdt[1], kdt[2], kdt[3]);
        *reinterpret_cast<float4*>(cons + CS_KDQD + kmajor_f32_off(32 + tok, 4 * lane, 8192)) = make_float4(qdt[0], qdt[1], qdt[2], qdt[3]);
      }
    }
    PROF_STAMP(2, 27);
    fence_proxy_async();                                  // this thread's reads / writes of the g region precede its refill
    named_bar_sync(bar_id, PREP_THREADS);
    if (lane == 0) mbar_arrive(x.bar(B_G_EMPTY + s));     // the gate tile may be refilled: step C does not read it
    PROF_STAMP(2, 28);

    // ---- C: one 16x16 block of A = kd' ki'^T (warps 0-3) or M = qd' ki'^T (warps 4-7) per warp
    {
      const int which = pw >> 2, rb = (pw >> 1) & 1, cb = pw & 1;
      const int g = lane >> 2, t = lane & 3;
      const int i0 = 16 * rb + g, i1 = i0 + 8;
      float acc[2][4];
#pragma unroll
      for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
      if (!(rb == 0 && cb == 1)) {
        const uint32_t a_tile = smem_u32(raw + (which ? RAW_Q : RAW_K));
        const uint32_t b_tile = smem_u32(kis_tile);
        const int a_row = 16 * rb + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int b_row = 16 * cb + 8 * (lane >> 4) + (lane & 7);
#pragma unroll
        for (int kt = 0; kt < 8; kt++) {
          uint32_t a[4], b[4];
          ldmatrix_x4(a, a_tile + rawtile_off(a_row, (2 * kt + (lane >> 4)) * 8));
          ldmatrix_x4(b, b_tile + rawtile_off(b_row, (2 * kt + ((lane >> 3) & 1)) * 8));
          mma_bf16(acc[0], a, b[0], b[1]);
          mma_bf16(acc[1], a, b[2], b[3]);
        }
      }
      PROF_STAMP(2, 15);
      if (which == 0) {
        x.wait(B_L_EMPTY + s, par ^ 1, E_PREP);
        float* Lsm = reinterpret_cast<float*>(x.smem + OFF_L) + s * 1024;
        const float b0 = beta_s[i0], b1 = beta_s[i1];
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
          const int j = 16 * cb + 8 * nt + 2 * t;
          *reinterpret_cast<float2*>(Lsm + i0 * C + j) = make_float2((j < i0) ? acc[nt][0] * b0 : 0.0f, (j + 1 < i0) ? acc[nt][1] * b0 : 0.0f);
          *reinterpret_cast<float2*>(Lsm + i1 * C + j) = make_float2((j < i1) ? acc[nt][2] * b1 : 0.0f, (j + 1 < i1) ? acc[nt][3] * b1 : 0.0f);
        }
        if (pw == 0) reinterpret_cast<float*>(x.smem + OFF_LBETA)[s * 32 + lane] = beta_s[lane];
        __syncwarp();
        if (lane == 0) mbar_arrive(x.bar(B_L_FULL + s));      // the inverse of this chunk may start
      }
      PROF_STAMP(2, 16);
      // ---- D: the operands of MMA3 go out once the tensor core has released the rest of the stage
      x.wait(B_CONS_EMPTY + s, par ^ 1, E_PREP);
      PROF_STAMP(2, 17);
#pragma unroll
      for (int tt = 0; tt < 4; tt++)
        *reinterpret_cast<float4*>(cons + CS_KR + mnmajor_f32_off(4 * lane, 4 * pw + tt, 512, 2048)) =
            make_float4(krr[tt][0], krr[tt][1], krr[tt][2], krr[tt][3]);
      if (which == 1) {
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
          const int j = 16 * cb + 8 * nt + 2 * t;
          *reinterpret_cast<float2*>(cons + CS_M + kmajor_f32_off(i0, j, 0)) =
              make_float2((j <= i0) ? acc[nt][0] : 0.0f, (j + 1 <= i0) ? acc[nt][1] : 0.0f);
          *reinterpret_cast<float2*>(cons + CS_M + kmajor_f32_off(i1, j, 0)) =
              make_float2((j <= i1) ? acc[nt][2] : 0.0f, (j + 1 <= i1) ? acc[nt][3] : 0.0f);
        }
      }
    }
    PROF_STAMP(2, 29);
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(x.bar(B_P1_FULL + s));
      mbar_arrive(x.bar(B_QK_EMPTY + s));        // the q / k tiles are no longer read
    }
  }
}

// ------------------------------------------------------------------------------------------------ inverse warps
// T = (I + L)^-1 for the strictly lower triangular fp32 L [32][32] of a chunk, in place in L's buffer, by one warp:
//   1. the two 16x16 diagonal blocks by forward substitution in fp32 registers, one half-warp per block, lane = column
//      (16 dependent rows instead of 32);
//   2. the off-diagonal block T10 = -T11 (L10 T00) as two 16x16x16 products on mma.sync (tf32 operands, fp32
//      accumulation; T is consumed as a tf32 / bf16 tensor-core operand anyway).
// Then Tb = T diag(beta) goes out as the tf32 and bf16 operand tiles of MMA2.
__device__ __forceinline__ void mm16_tf32(float (&acc)[2][4], const float* A, const float* B, int lane) {
  // acc[nt] (16 x 8) += A[16][16] * B[16][16], both row-major with a row stride of 32 floats
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int kt = 0; kt < 2; kt++) {
    const uint32_t a[4] = {__float_as_uint(A[g * C + 8 * kt + t]), __float_as_uint(A[(g + 8) * C + 8 * kt + t]),
                           __float_as_uint(A[g * C + 8 * kt + t + 4]), __float_as_uint(A[(g + 8) * C + 8 * kt + t + 4])};
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
      mma_tf32(acc[nt], a, __float_as_uint(B[(8 * kt + t) * C + 8 * nt + g]), __float_as_uint(B[(8 * kt + t + 4) * C + 8 * nt + g]));
  }
}

__device__ void role_inverse(const Ctx& x, int which, int lane) {
  const int blk = lane >> 4, cl = lane & 15;
  const int g = lane >> 2, t = lane & 3;
#pragma unroll 1
  for (int c = which; c < x.nchunks; c += 2) {
    const int s = c & 1;
    const uint32_t par = (uint32_t)((c >> 1) & 1);
    // Everything that does not depend on this chunk's L comes first, while the warp would only wait for L anyway (the
    // v tile and the release of the stage by MMA3 of the chunk two back are normally long there): after the inversion
    // only the operand write-out remains between L and MMA2.
    // The v tile of a partial last chunk holds another sequence's rows (or worse) past the end of the run: zero them
    // so that they cannot poison MMA2 (their Tb columns are zero, but 0 * NaN is NaN).  This warp observes every
    // phase of the v barrier of its stage, so the wait cannot be satisfied by an older phase, and MMA2 waits for this
    // warp's INV_FULL arrival.
    x.wait(B_V_FULL + s, par, E_INV);
    {
      const int nvalid = min(C, x.len - c * C);
      if (nvalid < C) {
        uint8_t* vt = x.smem + OFF_CONS + s * CS_STAGE + CS_V;
        for (int i = lane; i < (C - nvalid) * 16; i += 32) {     // whole 128-byte lines of both 64-channel halves
          const int row = nvalid + (i >> 4), piece = i & 15;
          *reinterpret_cast<uint4*>(vt + (piece >> 3) * 4096 + row * 128 + (piece & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    x.wait(B_CONS_EMPTY + s, par ^ 1, E_INV);
    x.wait(B_L_FULL + s, par, E_INV);
    float* Lsm = reinterpret_cast<float*>(x.smem + OFF_L) + s * 1024;
    PROF_BEGIN;
    // ---- 1: diagonal blocks
    {
      const float* Lb = Lsm + blk * 16 * C + blk * 16;
      float Tc[16];
#pragma unroll
      for (int i = 0; i < 16; i++) {
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
        for (int j = 0; j + 3 < i; j += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(Lb + i * C + j);
          a0 = fmaf(l4.x, Tc[j], a0);
          a1 = fmaf(l4.y, Tc[j + 1], a1);
          a2 = fmaf(l4.z, Tc[j + 2], a2);
          a3 = fmaf(l4.w, Tc[j + 3], a3);
        }
#pragma unroll
        for (int j = i & ~3; j < i; j++) a0 = fmaf(Lb[i * C + j], Tc[j], a0);
        Tc[i] = ((i == cl) ? 1.0f : 0.0f) - ((a0 + a1) + (a2 + a3));
      }
      __syncwarp();                                   // every lane has read its diagonal block
      float* Tb_ = Lsm + blk * 16 * C + blk * 16;
#pragma unroll
      for (int i = 0; i < 16; i++) Tb_[i * C + cl] = Tc[i];
    }
    __syncwarp();
    // ---- 2: T10 = -T11 (L10 T00), in place in the (1,0) block
    {
      float* L10 = Lsm + 16 * C;
      float acc[2][4];
#pragma unroll
      for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
      mm16_tf32(acc, L10, Lsm, lane);                 // X = L10 T00
      __syncwarp();                                   // L10 fully read
#pragma unroll
      for (int nt = 0; nt < 2; nt++) {
        *reinterpret_cast<float2*>(L10 + g * C + 8 * nt + 2 * t) = make_float2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<float2*>(L10 + (g + 8) * C + 8 * nt + 2 * t) = make_float2(acc[nt][2], acc[nt][3]);
        acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
      }
      __syncwarp();
      mm16_tf32(acc, Lsm + 16 * C + 16, L10, lane);   // T11 X
      __syncwarp();                                   // X fully read
#pragma unroll
      for (int nt = 0; nt < 2; nt++) {
        *reinterpret_cast<float2*>(L10 + g * C + 8 * nt + 2 * t) = make_float2(-acc[nt][0], -acc[nt][1]);
        *reinterpret_cast<float2*>(L10 + (g + 8) * C + 8 * nt + 2 * t) = make_float2(-acc[nt][2], -acc[nt][3]);
      }
    }
    __syncwarp();
    const float* lbeta = reinterpret_cast<const float*>(x.smem + OFF_LBETA) + s * 32;
    PROF_STAMP(3, 26);
    uint8_t* tb = x.smem + OFF_CONS + s * CS_STAGE + CS_TB;
    uint8_t* tbh = x.smem + OFF_TBH + s * 2048;
    // Tb = T diag(beta): lane = row; eight columns (one 16-byte bf16 chunk, two 16-byte tf32 chunks) per step, the
    // column group rotated by the lane so that the wide loads and stores of a quarter-warp spread over the banks.
#pragma unroll
    for (int jj = 0; jj < 4; jj++) {
      const int c0 = 8 * ((jj + lane) & 3);
      const float4 ta = *reinterpret_cast<const float4*>(Lsm + lane * C + c0);
      const float4 tc = *reinterpret_cast<const float4*>(Lsm + lane * C + c0 + 4);
      const float4 ba = *reinterpret_cast<const float4*>(lbeta + c0);
      const float4 bb = *reinterpret_cast<const float4*>(lbeta + c0 + 4);
      const float4 va = make_float4(ta.x * ba.x, ta.y * ba.y, ta.z * ba.z, ta.w * ba.w);
      const float4 vb = make_float4(tc.x * bb.x, tc.y * bb.y, tc.z * bb.z, tc.w * bb.w);
      *reinterpret_cast<float4*>(tb + kmajor_f32_off(lane, c0, 0)) = va;
      *reinterpret_cast<float4*>(tb + kmajor_f32_off(lane, c0 + 4, 0)) = vb;
      *reinterpret_cast<uint4*>(tbh + kmajor_b16_sw64_off(lane, c0)) =
          make_uint4(pack_bf16(va.x, va.y), pack_bf16(va.z, va.w), pack_bf16(vb.x, vb.y), pack_bf16(vb.z, vb.w));
    }
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(x.bar(B_INV_FULL + s));
      mbar_arrive(x.bar(B_L_EMPTY + s));
    }
  }
}

// ------------------------------------------------------------------------------------------------ MMA issuer
// Runs on ALL lanes of warp 0 with warp-uniform values only; one elected lane issues the tensor-core instructions
// (predicated inside the asm).  Keeping the control flow convergent lets the compiler hold descriptors, tensor-memory
// addresses and barrier addresses in uniform registers, which is what makes issuing ~34 small MMAs per chunk cheap.
__device__ void role_mma(const Ctx& x, uint32_t tmem_any, bool v_zero_any) {
  const uint32_t go = elect_one();
  const uint32_t tmem = __shfl_sync(0xffffffffu, tmem_any, 0);
  const bool v_zero = __shfl_sync(0xffffffffu, (int)v_zero_any, 0) != 0;
  const int nchunks = __shfl_sync(0xffffffffu, x.nchunks, 0);
  const uint32_t sb = smem_u32(x.smem);
  constexpr uint32_t ID1 = make_idesc(FMT_TF32, 128, 64, 0, 0, 0);
  constexpr uint32_t ID2A = make_idesc(FMT_BF16, 128, 32, 1, 0, 0);
  constexpr uint32_t ID2B = make_idesc(FMT_TF32, 128, 32, 0, 0, 1);
  constexpr uint32_t ID3A = make_idesc(FMT_TF32, 128, 128, 0, 1, 0);
  constexpr uint32_t ID3B = make_idesc(FMT_TF32, 128, 32, 0, 0, 0);
  const uint32_t tS = tmem + TM_S;
  // Descriptors of stage 0, built once; a stage or K step only moves the 14-bit start-address field (units of 16
  // bytes), so every other descriptor is one 64-bit add away.
  const uint64_t d_kdqd = make_sdesc(sb + OFF_CONS + CS_KDQD, 16, 1024, LAYOUT_SW128);
  const uint64_t d_v = make_sdesc(sb + OFF_CONS + CS_V, 4096, 1024, LAYOUT_SW128);
  const uint64_t d_tbh = make_sdesc(sb + OFF_TBH, 16, 512, LAYOUT_SW64);
  const uint64_t d_tb = make_sdesc(sb + OFF_CONS + CS_TB, 16, 1024, LAYOUT_SW128);
  const uint64_t d_kr = make_sdesc(sb + OFF_CONS + CS_KR, 512, 2048, LAYOUT_SW128_BASE32B);
  const uint64_t d_m = make_sdesc(sb + OFF_CONS + CS_M, 16, 1024, LAYOUT_SW128);
  x.wait(B_S_READY, 0, E_MMA, 0);                  // initial state is in tensor memory
#pragma unroll 1
  for (int c = 0; c < nchunks; c++) {
    const int s = c & 1;
    const uint32_t par = (uint32_t)((c >> 1) & 1);
    const uint64_t so = (uint64_t)(s * (CS_STAGE >> 4));          // stage offset in the start-address field
    const uint64_t so_tbh = (uint64_t)(s * (2048 >> 4));
    const uint32_t tWO = tmem + TM_WO + 64 * s;
    const uint32_t tU = tmem + TM_U + 32 * s;             // U alternates too: MMA2 of the next chunk never overwrites
                                                          // columns that MMA3 of this chunk may still be reading
    x.wait(B_P1_FULL + s, par, E_MMA, 0);
    x.wait(B_O_EMPTY + s, par ^ 1, E_MMA, 0);
    tc_fence_after();
    PROF_BEGIN;
#pragma unroll
    for (int ks = 0; ks < 16; ks++)
      mma_ts_tf32_pred(tWO, tS + 8 * ks, d_kdqd + so + (uint64_t)(((ks >> 2) * 8192 + (ks & 3) * 32) >> 4), ID1, ks > 0, go);
    mma_commit_pred(x.bar(B_MMA1_DONE), go);              // the tensor-memory warps may rescale the state
    mma_commit_pred(x.bar(B_KDQD_EMPTY + s), go);         // [kd ; qd] of this stage may be rewritten
    PROF_STAMP(4, 26);
    x.wait(B_INV_FULL + s, par, E_MMA, 0);
    x.wait(B_V_FULL + s, par, E_MMA, 0);
    tc_fence_after();
    if (!v_zero) {
#pragma unroll
      for (int ks = 0; ks < 2; ks++)
        mma_ss_f16_pred(tU, d_v + so + (uint64_t)((2 * ks * 1024) >> 4), d_tbh + so_tbh + (uint64_t)((ks * 32) >> 4), ID2A, ks > 0, go);
    }
#pragma unroll
    for (int ks = 0; ks < 4; ks++)
      mma_ts_tf32_pred(tU, tWO + 8 * ks, d_tb + so + (uint64_t)((ks * 32) >> 4), ID2B, (ks > 0) || !v_zero, go);
    PROF_STAMP(4, 27);
    mma_commit_pred(x.bar(B_V_EMPTY + s), go);            // the v tile may be refilled once MMA2 has read it
#pragma unroll
    for (int ks = 0; ks < 4; ks++)                        // O += U M^T does not touch the state: issued before the wait
      mma_ts_tf32_pred(tWO + 32, tU + 8 * ks, d_m + so + (uint64_t)((ks * 32) >> 4), ID3B, 1, go);
    mma_commit_pred(x.bar(B_O_FULL + s), go);
    x.wait(B_S_READY, (uint32_t)((c + 1) & 1), E_MMA, 0); // decay St <- St diag(2^G31) finished
    tc_fence_after();
#pragma unroll
    for (int ks = 0; ks < 4; ks++)
      mma_ts_tf32_pred(tS, tU + 8 * ks, d_kr + so + (uint64_t)((ks * 4096) >> 4), ID3A, 1, go);
    PROF_STAMP(4, 28);
    mma_commit_pred(x.bar(B_CONS_EMPTY + s), go);
    PROF_STAMP(4, 29);
  }
  mma_commit_pred(x.bar(B_MMA1_DONE), go);         // the final state is complete
  mma_commit_pred(x.bar(B_DRAIN), go);
  // every tensor-core instruction has retired before tensor memory is freed, also after a give-up elsewhere
  if (!mbar_wait_drain(x.bar(B_DRAIN), 0, x.abort_flag)) atomicCAS(const_cast<int*>(x.abort_flag), 0, E_DRAIN + B_DRAIN);
}

// ------------------------------------------------------------------------------------------------ tensor-memory warps
template <typename OutT>
__device__ __forceinline__ void store_row_piece(OutT* dst_head, int key_first, int v, int col0, const uint32_t (&r)[32]);

template <>
__device__ __forceinline__ void store_row_piece<float>(float* dst, int key_first, int v, int col0, const uint32_t (&r)[32]) {
  if (!key_first) {
    float4* d = reinterpret_cast<float4*>(dst + v * D + col0);
#pragma unroll
    for (int i = 0; i < 8; i++)
      d[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
  } else {
#pragma unroll
    for (int i = 0; i < 32; i++) dst[(col0 + i) * D + v] = __uint_as_float(r[i]);
  }
}
template <>
__device__ __forceinline__ void store_row_piece<__nv_bfloat16>(__nv_bfloat16* dst, int key_first, int v, int col0, const uint32_t (&r)[32]) {
  if (!key_first) {
    uint4* d = reinterpret_cast<uint4*>(dst + v * D + col0);
#pragma unroll
    for (int i = 0; i < 4; i++)
      d[i] = make_uint4(pack_bf16(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1])), pack_bf16(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3])),
                        pack_bf16(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5])), pack_bf16(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7])));
  } else {
#pragma unroll
    for (int i = 0; i < 32; i++) dst[(col0 + i) * D + v] = __float2bfloat16_rn(__uint_as_float(r[i]));
  }
}

// State columns [64 hf, 64 hf + 64) of this warp's 32 value rows: tensor memory -> final-state tensor and / or
// checkpoint row (either may be null).
template <int KF>
__device__ __noinline__ void store_state_rows(uint32_t tS, float* dst, void* ck, int ck_is_bf16, int v, int hf) {
#pragma unroll 1
  for (int j = 0; j < 2; j++) {
    const int col0 = 64 * hf + 32 * j;
    uint32_t r[32];
    tmem_ld32(tS + 32 * j, r);
    tmem_wait_ld();
    if (ck != nullptr) {
      if (ck_is_bf16) store_row_piece<__nv_bfloat16>(reinterpret_cast<__nv_bfloat16*>(ck), KF, v, col0, r);
      else store_row_piece<float>(reinterpret_cast<float*>(ck), KF, v, col0, r);
    }
    if (dst != nullptr) store_row_piece<float>(dst, KF, v, col0, r);
  }
}

// r[i] <- r[i] * d[i] for 16 consecutive state columns (d in shared memory, 16-byte aligned)
__device__ __forceinline__ void scale16(uint32_t (&r)[16], const float* d) {
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float4 d4 = *reinterpret_cast<const float4*>(d + 4 * i);
    const float2 lo = mul2(make_float2(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1])), make_float2(d4.x, d4.y));
    const float2 hi = mul2(make_float2(__uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])), make_float2(d4.z, d4.w));
    r[4 * i] = __float_as_uint(lo.x); r[4 * i + 1] = __float_as_uint(lo.y);
    r[4 * i + 2] = __float_as_uint(hi.x); r[4 * i + 3] = __float_as_uint(hi.y);
  }
}

// Eight warps own the tensor-memory traffic that goes through registers: warp (quarter q, half hf) serves the 32
// value rows [32 q, 32 q + 32) (the tensor-memory lanes a warp with id % 4 == q may touch) and, of those, the state
// columns [64 hf, 64 hf + 64) and the output tokens [16 hf, 16 hf + 16) of every chunk.  Per chunk:
//   wait MMA1 done -> (checkpoint row if due) -> St <- St diag(2^G31) for its columns -> signal S_READY        (on the chain)
//   wait MMA3 done -> O columns -> registers -> release the O buffer -> bf16 -> global                         (off the chain)
// plus the initial state load and the final state store for its columns.
template <int KF>
__device__ void role_tmem(const ChunkParams& p, const Task& task, const Ctx& x, uint32_t tmem, int quarter, int hf, int lane) {
  const int v = 32 * quarter + lane;
  const uint32_t lane_base = (uint32_t)(32 * quarter) << 16;
  const uint32_t tS = tmem + TM_S + lane_base + 64 * hf;
  // ---- initial state -> tensor memory
#pragma unroll 1
  for (int j = 0; j < 2; j++) {
    const int col0 = 64 * hf + 32 * j;
    uint32_t r[32];
    if (task.flags & (TF_INIT_ZERO | TF_INIT_IDENTITY)) {
      const float one = (task.flags & TF_INIT_IDENTITY) ? 1.0f : 0.0f;
#pragma unroll
      for (int i = 0; i < 32; i++) r[i] = __float_as_uint((col0 + i == v) ? one : 0.0f);
    } else {
      const float* src = task.src + (size_t)x.h * STATE_ELEMS;
      if (!KF) {
        const float4* s4 = reinterpret_cast<const float4*>(src + v * D + col0);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float4 f = s4[i];
          r[4 * i] = __float_as_uint(f.x); r[4 * i + 1] = __float_as_uint(f.y); r[4 * i + 2] = __float_as_uint(f.z); r[4 * i + 3] = __float_as_uint(f.w);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; i++) r[i] = __float_as_uint(src[(col0 + i) * D + v]);
      }
    }
    tmem_st32(tS + 32 * j, r);
  }
  tmem_wait_st();
  tc_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive(x.bar(B_S_READY));

  __nv_bfloat16* obase = ((task.flags & TF_OUT_AUX) ? p.out_aux : p.out) + (long long)x.h * D + v;
#pragma unroll 1
  for (int c = 0; c <= x.nchunks; c++) {
    x.wait(B_MMA1_DONE, (uint32_t)(c & 1), E_SCALE);
    tc_fence_after();
    const bool last = c == x.nchunks;
    const bool ck = !last && task.ck != nullptr && p.ck_every_chunks > 0 && (c % p.ck_every_chunks) == 0;
    const float* dec = reinterpret_cast<const float*>(x.smem + OFF_DEC) + (c & 3) * D;
    long long ck_off = 0;
    if (ck) ck_off = (long long)(c / p.ck_every_chunks) * p.ck_row_stride + (long long)x.h * STATE_ELEMS;
    // Checkpoint rows and the final state leave tensor memory through an out-of-line routine, so that their register
    // needs do not weigh on the per-chunk path below.
    if (ck || last) {
      float* dst = (last && task.dst != nullptr) ? task.dst + (size_t)x.h * STATE_ELEMS : nullptr;
      void* ckp = nullptr;
      if (ck) ckp = p.ck_is_bf16 ? static_cast<void*>(reinterpret_cast<__nv_bfloat16*>(task.ck) + ck_off)
                                 : static_cast<void*>(reinterpret_cast<float*>(task.ck) + ck_off);
      if (KF && (task.flags & TF_DST_VF)) store_state_rows<0>(tS, dst, ckp, p.ck_is_bf16, v, hf);   // transition maps
      else store_state_rows<KF>(tS, dst, ckp, p.ck_is_bf16, v, hf);
    }
    if (last) break;
    {
      // The decay sits on the serial chain MMA1 -> decay -> MMA3 -> MMA1 of the next chunk: four 16-column pieces,
      // the tensor-memory load of a piece in flight while the previous one is scaled and stored.
      const float* dcol = dec + 64 * hf;
      uint32_t a[16], b[16], e[16];
      tmem_ld16(tS, a);
      tmem_ld16(tS + 16, b);
      tmem_wait_ld();
      scale16(a, dcol);
      tmem_st16(tS, a);
      tmem_ld16(tS + 32, e);
      scale16(b, dcol + 16);
      tmem_st16(tS + 16, b);
      tmem_ld16(tS + 48, a);
      tmem_wait_ld();
      scale16(e, dcol + 32);
      tmem_st16(tS + 32, e);
      scale16(a, dcol + 48);
      tmem_st16(tS + 48, a);
    }
    tmem_wait_st();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(x.bar(B_S_READY));

    // ---- output rows of this chunk
    const int s = c & 1;
    x.wait(B_O_FULL + s, (uint32_t)((c >> 1) & 1), E_EPI);
    tc_fence_after();
    uint32_t o[16];
    tmem_ld16(tmem + TM_WO + 64 * s + 32 + 16 * hf + lane_base, o);
    tmem_wait_ld();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(x.bar(B_O_EMPTY + s));
    if (!(task.flags & TF_NO_OUT)) {
      const int nvalid = min(C, x.len - c * C);
      __nv_bfloat16* orow = obase + (x.t0 + (long long)c * C + 16 * hf) * p.ldo;
      if (nvalid == C) {
#pragma unroll
        for (int i = 0; i < 16; i++) orow[(long long)i * p.ldo] = __float2bfloat16_rn(__uint_as_float(o[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 16; i++)
          if (16 * hf + i < nvalid) orow[(long long)i * p.ldo] = __float2bfloat16_rn(__uint_as_float(o[i]));
      }
    }
  }
}

// ================================================================================================ dual-chain tasks
// Context parallelism and the cuts of long sequences need, for a token segment whose entering state is not known yet,
// TWO chains over the same tokens: chain L from S = 0 with the real v (o_loc, S_loc) and chain Tr from S = I with v = 0
// (Qt, P).  Everything the preparation warps, the loader and the inverse warps produce is the same for both, and the
// tensor pipe is busy a quarter of the time, so a task flagged TF_DUAL runs both chains over ONE operand preparation: a
// second state in tensor-memory columns 128-255, each MMA group issued twice, the tensor-memory warps serving both
// states (function of the reference's dual kernel, kda/b200/csrc/w3/base/cake_dual/kda_m128.cu:821-823,
// kda/b200/csrc/w3/base/dual.py:1-4).  The issuer and the tensor-memory warps have roles of their own for such a task
// (chosen once per CTA, so a launch mixes plain and dual tasks at no cost to the plain ones); the other roles do not
// know the difference.
// Tensor memory of a dual task: S_L 0-127, S_T 128-255, [W | O] of L 256-319, of T 320-383 (one buffer per chain: the
// other chain's work hides the read-out), U of L 384-447, of T 448-511 (two stages each).

__device__ void role_mma_dual(const Ctx& x, uint32_t tmem_any, bool v_zero_any) {
  const uint32_t go = elect_one();
  const uint32_t tmem = __shfl_sync(0xffffffffu, tmem_any, 0);
  const bool v_zero = __shfl_sync(0xffffffffu, (int)v_zero_any, 0) != 0;
  const int nchunks = __shfl_sync(0xffffffffu, x.nchunks, 0);
  const uint32_t sb = smem_u32(x.smem);
  constexpr uint32_t ID1 = make_idesc(FMT_TF32, 128, 64, 0, 0, 0);
  constexpr uint32_t ID2A = make_idesc(FMT_BF16, 128, 32, 1, 0, 0);
  constexpr uint32_t ID2B = make_idesc(FMT_TF32, 128, 32, 0, 0, 1);
  constexpr uint32_t ID3A = make_idesc(FMT_TF32, 128, 128, 0, 1, 0);
  constexpr uint32_t ID3B = make_idesc(FMT_TF32, 128, 32, 0, 0, 0);
  const uint64_t d_kdqd = make_sdesc(sb + OFF_CONS + CS_KDQD, 16, 1024, LAYOUT_SW128);
  const uint64_t d_v = make_sdesc(sb + OFF_CONS + CS_V, 4096, 1024, LAYOUT_SW128);
  const uint64_t d_tbh = make_sdesc(sb + OFF_TBH, 16, 512, LAYOUT_SW64);
  const uint64_t d_tb = make_sdesc(sb + OFF_CONS + CS_TB, 16, 1024, LAYOUT_SW128);
  const uint64_t d_kr = make_sdesc(sb + OFF_CONS + CS_KR, 512, 2048, LAYOUT_SW128_BASE32B);
  const uint64_t d_m = make_sdesc(sb + OFF_CONS + CS_M, 16, 1024, LAYOUT_SW128);
  const uint32_t tS0 = tmem + TD_S0, tS1 = tmem + TD_S1, tWO1 = tmem + TD_WO1;
  x.wait(B_S_READY, 0, E_MMA, 0);                  // initial states are in tensor memory
  x.wait(B_S_READY_T, 0, E_MMA, 0);
#pragma unroll 1
  for (int c = 0; c < nchunks; c++) {
    const int s = c & 1;
    const uint32_t par = (uint32_t)((c >> 1) & 1), cpar = (uint32_t)(c & 1);
    const uint64_t so = (uint64_t)(s * (CS_STAGE >> 4));
    const uint64_t so_tbh = (uint64_t)(s * (2048 >> 4));
    const uint32_t tU0 = tmem + TD_U0 + 32 * s, tU1 = tmem + TD_U1 + 32 * s;
    // [W | O]: one buffer per chain (one phase per chunk), not per stage as in the single-chain role
    const uint32_t tWO0 = tmem + TD_WO0;
    x.wait(B_P1_FULL + s, par, E_MMA, 0);
    x.wait(B_O_EMPTY + 0, cpar ^ 1, E_MMA, 0);
    tc_fence_after();
#pragma unroll
    for (int ks = 0; ks < 16; ks++)
      mma_ts_tf32_pred(tWO0, tS0 + 8 * ks, d_kdqd + so + (uint64_t)(((ks >> 2) * 8192 + (ks & 3) * 32) >> 4), ID1, ks > 0, go);
    mma_commit_pred(x.bar(B_MMA1_DONE), go);
    x.wait(B_O_EMPTY + 1, cpar ^ 1, E_MMA, 0);
    tc_fence_after();
#pragma unroll
    for (int ks = 0; ks < 16; ks++)
      mma_ts_tf32_pred(tWO1, tS1 + 8 * ks, d_kdqd + so + (uint64_t)(((ks >> 2) * 8192 + (ks & 3) * 32) >> 4), ID1, ks > 0, go);
    mma_commit_pred(x.bar(B_MMA1_DONE_T), go);
    mma_commit_pred(x.bar(B_KDQD_EMPTY + s), go);
    x.wait(B_INV_FULL + s, par, E_MMA, 0);
    x.wait(B_V_FULL + s, par, E_MMA, 0);
    tc_fence_after();
    if (!v_zero) {
#pragma unroll
      for (int ks = 0; ks < 2; ks++)
        mma_ss_f16_pred(tU0, d_v + so + (uint64_t)((2 * ks * 1024) >> 4), d_tbh + so_tbh + (uint64_t)((ks * 32) >> 4), ID2A, ks > 0, go);
    }
#pragma unroll
    for (int ks = 0; ks < 4; ks++)
      mma_ts_tf32_pred(tU0, tWO0 + 8 * ks, d_tb + so + (uint64_t)((ks * 32) >> 4), ID2B, (ks > 0) || !v_zero, go);
#pragma unroll
    for (int ks = 0; ks < 4; ks++)                      // the transition chain has v = 0: U = - W Tb^T
      mma_ts_tf32_pred(tU1, tWO1 + 8 * ks, d_tb + so + (uint64_t)((ks * 32) >> 4), ID2B, ks > 0, go);
    mma_commit_pred(x.bar(B_V_EMPTY + s), go);
#pragma unroll
    for (int ks = 0; ks < 4; ks++)
      mma_ts_tf32_pred(tWO0 + 32, tU0 + 8 * ks, d_m + so + (uint64_t)((ks * 32) >> 4), ID3B, 1, go);
    mma_commit_pred(x.bar(B_O_FULL + 0), go);
#pragma unroll
    for (int ks = 0; ks < 4; ks++)
      mma_ts_tf32_pred(tWO1 + 32, tU1 + 8 * ks, d_m + so + (uint64_t)((ks * 32) >> 4), ID3B, 1, go);
    mma_commit_pred(x.bar(B_O_FULL + 1), go);
    x.wait(B_S_READY, (uint32_t)((c + 1) & 1), E_MMA, 0);
    tc_fence_after();
#pragma unroll
    for (int ks = 0; ks < 4; ks++)
      mma_ts_tf32_pred(tS0, tU0 + 8 * ks, d_kr + so + (uint64_t)((ks * 4096) >> 4), ID3A, 1, go);
    x.wait(B_S_READY_T, (uint32_t)((c + 1) & 1), E_MMA, 0);
    tc_fence_after();
#pragma unroll
    for (int ks = 0; ks < 4; ks++)
      mma_ts_tf32_pred(tS1, tU1 + 8 * ks, d_kr + so + (uint64_t)((ks * 4096) >> 4), ID3A, 1, go);
    mma_commit_pred(x.bar(B_CONS_EMPTY + s), go);
  }
  mma_commit_pred(x.bar(B_MMA1_DONE), go);         // the final states are complete
  mma_commit_pred(x.bar(B_MMA1_DONE_T), go);
  mma_commit_pred(x.bar(B_DRAIN), go);
  if (!mbar_wait_drain(x.bar(B_DRAIN), 0, x.abort_flag)) atomicCAS(const_cast<int*>(x.abort_flag), 0, E_DRAIN + B_DRAIN);
}

// St <- St diag(d) for this warp's 64 state columns (four 16-column pieces, the load of one in flight while the
// previous one is scaled and stored)
__device__ __forceinline__ void decay64(uint32_t tS, const float* dcol) {
  uint32_t a[16], b[16], e[16];
  tmem_ld16(tS, a);
  tmem_ld16(tS + 16, b);
  tmem_wait_ld();
  scale16(a, dcol);
  tmem_st16(tS, a);
  tmem_ld16(tS + 32, e);
  scale16(b, dcol + 16);
  tmem_st16(tS + 16, b);
  tmem_ld16(tS + 48, a);
  tmem_wait_ld();
  scale16(e, dcol + 32);
  tmem_st16(tS + 32, e);
  scale16(a, dcol + 48);
  tmem_st16(tS + 48, a);
  tmem_wait_st();
}

template <int KF>
__device__ void role_tmem_dual(const ChunkParams& p, const Task& task, const Ctx& x, uint32_t tmem, int quarter, int hf, int lane) {
  const int v = 32 * quarter + lane;
  const uint32_t lane_base = (uint32_t)(32 * quarter) << 16;
  const uint32_t tS0 = tmem + TD_S0 + lane_base + 64 * hf, tS1 = tmem + TD_S1 + lane_base + 64 * hf;
  // ---- initial states -> tensor memory: chain L as the task says, chain Tr the identity
#pragma unroll 1
  for (int ch = 0; ch < 2; ch++) {
#pragma unroll 1
    for (int j = 0; j < 2; j++) {
      const int col0 = 64 * hf + 32 * j;
      uint32_t r[32];
      if (ch == 1 || (task.flags & (TF_INIT_ZERO | TF_INIT_IDENTITY))) {
        const float one = (ch == 1 || (task.flags & TF_INIT_IDENTITY)) ? 1.0f : 0.0f;
#pragma unroll
        for (int i = 0; i < 32; i++) r[i] = __float_as_uint((col0 + i == v) ? one : 0.0f);
      } else {
        const float* src = task.src + (size_t)x.h * STATE_ELEMS;
        if (!KF) {
          const float4* s4 = reinterpret_cast<const float4*>(src + v * D + col0);
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const float4 f = s4[i];
            r[4 * i] = __float_as_uint(f.x); r[4 * i + 1] = __float_as_uint(f.y); r[4 * i + 2] = __float_as_uint(f.z); r[4 * i + 3] = __float_as_uint(f.w);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++) r[i] = __float_as_uint(src[(col0 + i) * D + v]);
        }
      }
      tmem_st32((ch ? tS1 : tS0) + 32 * j, r);
    }
    tmem_wait_st();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(x.bar(ch ? B_S_READY_T : B_S_READY));
  }

  // Output of a dual-chain task: TILE-MAJOR scratch, [chunk][head][row v][32 tokens] bf16, Qt tiles at task.ck and the
  // o_loc tiles `oloc_tile_offset` elements behind them.  A lane owns one row v of the tile and 16 of its tokens, so
  // its share is 32 contiguous bytes (two 16-byte stores) instead of sixteen 2-byte stores 2 ldo bytes apart: the
  // tensor-memory warps are the busiest role of a dual task, and the output rows were a quarter of their time.  The
  // fix-up pass reads the tiles as they are (8 KB contiguous each) and writes the final rows.
  __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(task.ck) + (size_t)x.h * (D * C) + v * C + 16 * hf;
#pragma unroll 1
  for (int c = 0; c <= x.nchunks; c++) {
    const bool last = c == x.nchunks;
    const float* dcol = reinterpret_cast<const float*>(x.smem + OFF_DEC) + (c & 3) * D + 64 * hf;
#pragma unroll 1
    for (int ch = 0; ch < 2; ch++) {
      x.wait(ch ? B_MMA1_DONE_T : B_MMA1_DONE, (uint32_t)(c & 1), E_SCALE);
      tc_fence_after();
      const uint32_t tS = ch ? tS1 : tS0;
      if (last) {
        // final states: chain L in the launch's layout, the transition map always value-first
        float* dst = ch ? task.dst2 : task.dst;
        if (dst != nullptr) {
          dst += (size_t)x.h * STATE_ELEMS;
          if (ch == 1 || !KF || (task.flags & TF_DST_VF)) store_state_rows<0>(tS, dst, nullptr, 0, v, hf);
          else store_state_rows<KF>(tS, dst, nullptr, 0, v, hf);
        }
      } else {
        decay64(tS, dcol);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(x.bar(ch ? B_S_READY_T : B_S_READY));
      }
    }
    if (last) break;
    // ---- output tiles of this chunk, chain L then chain Tr
#pragma unroll 1
    for (int ch = 0; ch < 2; ch++) {
      x.wait(B_O_FULL + ch, (uint32_t)(c & 1), E_EPI);       // one output buffer per chain (see role_mma_dual)
      tc_fence_after();
      uint32_t o[16];
      tmem_ld16(tmem + (ch ? TD_WO1 : TD_WO0) + 32 + 16 * hf + lane_base, o);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(x.bar(B_O_EMPTY + ch));
      if (!(task.flags & TF_NO_OUT)) {
        uint4* dst = reinterpret_cast<uint4*>(tiles + (ch ? 0 : p.oloc_tile_offset) + (size_t)c * p.H * (D * C));
        dst[0] = make_uint4(pack_bf16(__uint_as_float(o[0]), __uint_as_float(o[1])), pack_bf16(__uint_as_float(o[2]), __uint_as_float(o[3])),
                            pack_bf16(__uint_as_float(o[4]), __uint_as_float(o[5])), pack_bf16(__uint_as_float(o[6]), __uint_as_float(o[7])));
        dst[1] = make_uint4(pack_bf16(__uint_as_float(o[8]), __uint_as_float(o[9])), pack_bf16(__uint_as_float(o[10]), __uint_as_float(o[11])),
                            pack_bf16(__uint_as_float(o[12]), __uint_as_float(o[13])), pack_bf16(__uint_as_float(o[14]), __uint_as_float(o[15])));
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ kernel
template <int FE, int KF>
__global__ void __launch_bounds__(THREADS, 1) kda_chunk_umma_kernel(const ChunkParams p, const __grid_constant__ TmaMaps maps) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = tid >> 5;
  const int H = p.H;
  const int rank = blockIdx.x / H, h = blockIdx.x % H;

  // Launched as a programmatic dependent of the planner (its CTAs become resident while the planner still runs): wait
  // here until the planner's writes (status, task table) are visible.  A no-op for an ordinary launch.
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  const int nt_word = *p.n_tasks;
  if (nt_word & NT_ZERO_FILL) {   // rejected cu_seqlens: all sequences empty, output rows zero-filled
    const long long rows = p.T * H;
    for (long long r = blockIdx.x; r < rows; r += gridDim.x)
      if (tid < 16) reinterpret_cast<uint4*>(p.out + (r / H) * p.ldo + (r % H) * D)[tid] = make_uint4(0, 0, 0, 0);
  }
  if (rank >= (nt_word & (NT_ZERO_FILL - 1))) return;
  const Task task = p.tasks[rank];
  Ctx x;
  x.smem = smem;
  x.bars = smem_u32(smem + OFF_BAR);
  x.abort_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 8);
  x.h = h;
  x.len = task.len;
  x.nchunks = (task.len + C - 1) / C;
  x.t0 = task.t0;
#ifdef KDA_PROF
  x.prof = p.prof;
  const long long prof_t0 = clock64();
#endif

  const bool dual = (task.flags & TF_DUAL) != 0;   // both chains of a mapped segment in this task (see the dual-chain roles)
  if (x.nchunks == 0) {
    // empty run: the state passes through (source -> destination) without touching tensor memory; the transition map
    // of no tokens is the identity
    for (int ch = 0; ch < (dual ? 2 : 1); ch++) {
      float* dst = ch ? task.dst2 : task.dst;
      if (dst == nullptr) continue;
      dst += (size_t)h * STATE_ELEMS;
      const bool ident = ch == 1 || (task.flags & TF_INIT_IDENTITY);
      const float* src = (ch == 1 || (task.flags & (TF_INIT_ZERO | TF_INIT_IDENTITY))) ? nullptr : task.src + (size_t)h * STATE_ELEMS;
      if (src == dst) continue;
      for (int i = tid; i < STATE_ELEMS / 4; i += THREADS) {
        float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
        if (src != nullptr) f = reinterpret_cast<const float4*>(src)[i];
        else if (ident) {
          const int row = (4 * i) / D, col = (4 * i) % D;
          f = make_float4(row == col ? 1.f : 0.f, row == col + 1 ? 1.f : 0.f, row == col + 2 ? 1.f : 0.f, row == col + 3 ? 1.f : 0.f);
        }
        reinterpret_cast<float4*>(dst)[i] = f;
      }
    }
    return;
  }

  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
  volatile int* range_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 12);
  if (tid == 0) {
    *x.abort_flag = 0;
    *range_flag = 0;
    *reinterpret_cast<volatile unsigned long long*>(smem + OFF_MISC + 16) = p.wait_limit_ns ? p.wait_limit_ns : kWaitLimitNs;
  }
  if (warp == W_INV0) {
    // One lane per barrier (the issuer warp allocates tensor memory meanwhile): a task of one or two chunks notices the
    // forty serial initialisations.  Arrival counts: the eight warps of a preparation group or the eight tensor-memory
    // warps where a whole group signals, four for the L tile (half a group), one everywhere else.
    constexpr unsigned long long EIGHT = (3ull << B_G_EMPTY) | (3ull << B_P1_FULL) | (3ull << B_O_EMPTY) | (1ull << B_S_READY) |
                                         (3ull << B_QK_EMPTY) | (1ull << B_S_READY_T);
    static_assert(PREP_WARPS == 8, "arrival counts of the group barriers");
    for (int i = lane; i < NUM_BARS; i += 32) {
      int count = ((EIGHT >> i) & 1ull) ? 8 : 1;
      if (i == B_L_FULL || i == B_L_FULL + 1) count = PREP_WARPS / 2;
      // diagnostic switch: the v barriers expect one arrival more than they will ever get, so their waiters give up
      if ((i == B_V_FULL || i == B_V_FULL + 1) && (p.debug_flags & DBG_STALL_V_STREAM)) count = 2;
      mbar_init(x.bar(i), count);
    }
    fence_barrier_init();
  }
  if (warp == W_MMA) {
    tmem_alloc(smem_u32(tmem_slot), TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const bool v_zero = (task.flags & TF_V_ZERO) != 0;

  if (warp == W_MMA) {
    if (dual) role_mma_dual(x, tmem, v_zero);
    else role_mma(x, tmem, v_zero);
    __syncwarp();
  } else if (warp == W_INV0 || warp == W_INV0 + 1) {
    role_inverse(x, warp - W_INV0, lane);
  } else if (warp == W_LOAD) {
    role_loader<FE>(p, maps, x, lane);
    __syncwarp();
  } else if (warp < W_PREP0) {
    if (dual) role_tmem_dual<KF>(p, task, x, tmem, warp & 3, (warp - W_SCALE0) >> 2, lane);
    else role_tmem<KF>(p, task, x, tmem, warp & 3, (warp - W_SCALE0) >> 2, lane);
  } else {
    const int pt = tid - W_PREP0 * 32;
    role_prep<FE>(p, x, pt / PREP_THREADS, pt % PREP_THREADS);
  }

#ifdef KDA_PROF
  if (lane == 0 && blockIdx.x == 0 && x.prof != nullptr) {
    const int role = warp == W_MMA ? 4 : (warp <= 2 ? 3 : (warp == W_LOAD ? 1 : (warp < W_PREP0 ? 5 : 2)));
    atomicAdd(x.prof + role * 128 + 126, (unsigned long long)(clock64() - prof_t0));
    atomicAdd(x.prof + role * 128 + 127, 1ull);
  }
#endif
  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    if (*x.abort_flag != 0) atomicCAS(p.status + 2, 0, *x.abort_flag);
    if (*range_flag != 0) atomicOr(p.status, KDA_BIT_RANGE);
  }
  if (warp == W_MMA) tmem_dealloc(tmem, TM_COLS);
}

}  // namespace u

cudaError_t launch_chunk_umma(const ChunkParams& p, const TmaMaps& maps, int n_task_cap, cudaStream_t stream, bool after_planner) {
  // one instantiation per (front-end, state layout): smaller code per launch, and instruction-cache footprint is what
  // bounds this role-specialised kernel
  typedef void (*Kern)(const ChunkParams, const TmaMaps);
  static const Kern kerns[2][2] = {{u::kda_chunk_umma_kernel<0, 0>, u::kda_chunk_umma_kernel<0, 1>},
                                   {u::kda_chunk_umma_kernel<1, 0>, u::kda_chunk_umma_kernel<1, 1>}};
  static int attr_dev_mask = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(attr_dev_mask & (1 << (dev & 31)))) {
    for (int i = 0; i < 4; i++) {
      cudaError_t e = cudaFuncSetAttribute(kerns[i >> 1][i & 1], cudaFuncAttributeMaxDynamicSharedMemorySize, u::SMEM_BYTES);
      if (e != cudaSuccess) return e;
    }
    attr_dev_mask |= 1 << (dev & 31);
  }
  const long long blocks = (long long)n_task_cap * p.H;
  if (blocks <= 0) return cudaSuccess;
  // Chained behind the planner by programmatic dependent launch when it directly follows it in the stream (function
  // of kda/b200/csrc/w3/base/cake/launch_m128.cu:37-60): the launch latency hides under the planner.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(u::THREADS);
  cfg.dynamicSmemBytes = u::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = after_planner ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kerns[p.frontend ? 1 : 0][p.key_first ? 1 : 0], p, maps);
}

}  // namespace kda
