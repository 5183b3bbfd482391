// Fused KDA chunk kernel for sm_100a: one CTA walks the 32-token chunks of one (token run, head) task.
//
// Per chunk (value-first state St [V][K] fp32, G = inclusive cumulative log2-decay, r = G after token 15):
//   prep warps   gate + cumsum, L2 norm, decayed bf16 operand tiles
//                  kd = k 2^G, qd = scale q 2^G, kr = k 2^(G31-G)           (state products)
//                  kd' = k 2^(G-r), qd' = scale q 2^(G-r), ki' = k 2^(r-G)  (intra-chunk products; every exponent is
//                  bounded by the decay of at most 16 tokens, so nothing overflows)
//                A = tril(kd' ki'^T, -1) * beta_i,  M = tril(qd' ki'^T),  T = (I + A)^-1 by forward substitution,
//                Tb = T diag(beta)
//   state warps  Wt = St kd^T;  Rt = v^T - Wt;  Ut = Rt Tb^T;  Ot = St qd^T + Ut M^T;  St = St diag(2^G31) + Ut kr
// which is the chunked form of kda/b200/reference.py:30-37 (the reference kernel's own statement of it:
// kda/b200/csrc/w3/base/tiny/kda_tiny.cu:5-11).  Each of the 8 state warps owns 16 value rows of St in registers as
// mma.sync accumulator fragments, so the whole chain of a warp needs no cross-warp exchange; prep warps run one chunk
// ahead through double-buffered shared-memory tiles.  The two roles meet at one __syncthreads per chunk: there is no
// spin-wait anywhere in this kernel.
#include "kda_common.cuh"

namespace kda {

constexpr int STATE_WARPS = 8;
constexpr int PREP_WARPS = 4;
constexpr int PREP_THREADS = PREP_WARPS * 32;
constexpr int THREADS = (STATE_WARPS + PREP_WARPS) * 32;

// ---- shared memory map (bytes)
constexpr int RAW_G = 0, RAW_Q = 16384, RAW_K = 24576, RAW_STAGE = 32768;      // x2
constexpr int OFF_RAW = 0;
constexpr int OFF_V = OFF_RAW + 2 * RAW_STAGE;                                   // 3 x 8192
constexpr int CS_KD = 0, CS_QD = 8192, CS_KR = 16384, CS_TB = 24576, CS_MM = 26624, CS_DEC = 28672, CS_STAGE = 29696;
constexpr int OFF_CONS = OFF_V + 3 * 8192;                                       // x2
constexpr int OFF_G = OFF_CONS + 2 * CS_STAGE;                                   // fp32 [32][128]
constexpr int OFF_KDS = OFF_G + 16384;
constexpr int OFF_QDS = OFF_KDS + 8192;
constexpr int OFF_KIS = OFF_QDS + 8192;
constexpr int OFF_L = OFF_KIS + 8192;                                            // fp32 [32][32]
constexpr int OFF_FR = OFF_L + 4096;                                             // r, 2^r, 2^(G31-r): 3 x fp32[128]
constexpr int OFF_BETA = OFF_FR + 1536;                                          // fp32[32]
constexpr int OFF_SLAB = OFF_BETA + 128;                                         // 8 warps x 32 rows x 48 B
constexpr int SLAB_ROW = 48;
constexpr int SMEM_BYTES = OFF_SLAB + STATE_WARPS * 32 * SLAB_ROW;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");

// ------------------------------------------------------------------------------------------------ state I/O
__device__ __forceinline__ void load_state(float (&S)[16][4], const Task& task, int h, int key_first, int warp, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const int v0 = 16 * warp + g;
  if (task.flags & (TF_INIT_ZERO | TF_INIT_IDENTITY)) {
    const float one = (task.flags & TF_INIT_IDENTITY) ? 1.0f : 0.0f;
#pragma unroll
    for (int nt = 0; nt < 16; nt++) {
      const int k0 = 8 * nt + 2 * t;
      S[nt][0] = (v0 == k0) ? one : 0.0f;
      S[nt][1] = (v0 == k0 + 1) ? one : 0.0f;
      S[nt][2] = (v0 + 8 == k0) ? one : 0.0f;
      S[nt][3] = (v0 + 8 == k0 + 1) ? one : 0.0f;
    }
    return;
  }
  const float* src = task.src + (size_t)h * STATE_ELEMS;
  if (!key_first) {
#pragma unroll
    for (int nt = 0; nt < 16; nt++) {
      const float2 a = *reinterpret_cast<const float2*>(src + v0 * D + 8 * nt + 2 * t);
      const float2 b = *reinterpret_cast<const float2*>(src + (v0 + 8) * D + 8 * nt + 2 * t);
      S[nt][0] = a.x; S[nt][1] = a.y; S[nt][2] = b.x; S[nt][3] = b.y;
    }
  } else {
#pragma unroll
    for (int nt = 0; nt < 16; nt++) {
      const int k0 = 8 * nt + 2 * t;
      S[nt][0] = src[k0 * D + v0];
      S[nt][1] = src[(k0 + 1) * D + v0];
      S[nt][2] = src[k0 * D + v0 + 8];
      S[nt][3] = src[(k0 + 1) * D + v0 + 8];
    }
  }
}

template <typename OutT>
__device__ __forceinline__ void store_state_t(const float (&S)[16][4], OutT* dst, int key_first, int warp, int lane);

template <>
__device__ __forceinline__ void store_state_t<float>(const float (&S)[16][4], float* dst, int key_first, int warp, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const int v0 = 16 * warp + g;
  if (!key_first) {
#pragma unroll
    for (int nt = 0; nt < 16; nt++) {
      *reinterpret_cast<float2*>(dst + v0 * D + 8 * nt + 2 * t) = make_float2(S[nt][0], S[nt][1]);
      *reinterpret_cast<float2*>(dst + (v0 + 8) * D + 8 * nt + 2 * t) = make_float2(S[nt][2], S[nt][3]);
    }
  } else {
#pragma unroll
    for (int nt = 0; nt < 16; nt++) {
      const int k0 = 8 * nt + 2 * t;
      dst[k0 * D + v0] = S[nt][0];
      dst[(k0 + 1) * D + v0] = S[nt][1];
      dst[k0 * D + v0 + 8] = S[nt][2];
      dst[(k0 + 1) * D + v0 + 8] = S[nt][3];
    }
  }
}

template <>
__device__ __forceinline__ void store_state_t<__nv_bfloat16>(const float (&S)[16][4], __nv_bfloat16* dst, int key_first,
                                                              int warp, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const int v0 = 16 * warp + g;
  if (!key_first) {
#pragma unroll
    for (int nt = 0; nt < 16; nt++) {
      *reinterpret_cast<uint32_t*>(dst + v0 * D + 8 * nt + 2 * t) = pack_bf16(S[nt][0], S[nt][1]);
      *reinterpret_cast<uint32_t*>(dst + (v0 + 8) * D + 8 * nt + 2 * t) = pack_bf16(S[nt][2], S[nt][3]);
    }
  } else {
#pragma unroll
    for (int nt = 0; nt < 16; nt++) {
      const int k0 = 8 * nt + 2 * t;
      dst[k0 * D + v0] = __float2bfloat16_rn(S[nt][0]);
      dst[(k0 + 1) * D + v0] = __float2bfloat16_rn(S[nt][1]);
      dst[k0 * D + v0 + 8] = __float2bfloat16_rn(S[nt][2]);
      dst[(k0 + 1) * D + v0 + 8] = __float2bfloat16_rn(S[nt][3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ prep role
struct PrepCtx {
  int ptid, pw, lane;
  int h;
  long long t0;
  int len;
  float eA;        // exp(A_log[h])        (raw front-end)
  float dtb;       // dt_bias[h*128 + ptid] (raw front-end)
};

__device__ __forceinline__ void prep_issue_loads(const ChunkParams& p, const PrepCtx& x, uint8_t* smem, int chunk) {
  const int rs = chunk & 1, vs = chunk % 3;
  const int nvalid = min(C, x.len - chunk * C);
  const long long tok0 = x.t0 + (long long)chunk * C;
  uint8_t* raw = smem + OFF_RAW + rs * RAW_STAGE;
  const uint32_t graw = smem_u32(raw + RAW_G), qraw = smem_u32(raw + RAW_Q), kraw = smem_u32(raw + RAW_K);
  const uint32_t vdst = smem_u32(smem + OFF_V + vs * 8192);
  if (p.frontend == 1) {
    const float* g = reinterpret_cast<const float*>(p.g);
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int idx = x.ptid + PREP_THREADS * j, row = idx >> 5, ch = idx & 31;
      const bool ok = row < nvalid;
      const float* src = g + (tok0 + (ok ? row : 0)) * p.ldg + (long long)x.h * D + ch * 4;
      cp_async16(graw + row * 512 + ch * 16, src, ok ? 16 : 0);
    }
  } else {
    const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(p.g);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int idx = x.ptid + PREP_THREADS * j, row = idx >> 4, ch = idx & 15;
      const bool ok = row < nvalid;
      const __nv_bfloat16* src = g + (tok0 + (ok ? row : 0)) * p.ldg + (long long)x.h * D + ch * 8;
      cp_async16(graw + row * 256 + ch * 16, src, ok ? 16 : 0);
    }
  }
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int idx = x.ptid + PREP_THREADS * j, row = idx >> 4, ch = idx & 15;
    const bool ok = row < nvalid;
    const long long tok = tok0 + (ok ? row : 0);
    const int n = ok ? 16 : 0;
    cp_async16(qraw + row * 256 + ch * 16, p.q + tok * p.ldq + (long long)x.h * D + ch * 8, n);
    cp_async16(kraw + row * 256 + ch * 16, p.k + tok * p.ldk + (long long)x.h * D + ch * 8, n);
    cp_async16(vdst + row * 256 + ((ch ^ (row & 7)) << 4), p.v + tok * p.ldv + (long long)x.h * D + ch * 8, n);
  }
}

// beta of token `row` of `chunk`, activated; 0 beyond the end of the run
__device__ __forceinline__ float prep_load_beta(const ChunkParams& p, const PrepCtx& x, int chunk, int row) {
  const int nvalid = min(C, x.len - chunk * C);
  if (row >= nvalid) return 0.0f;
  const long long tok = x.t0 + (long long)chunk * C + row;
  if (p.frontend == 1) return reinterpret_cast<const float*>(p.beta)[tok * p.ldbeta + x.h];
  const float b = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.beta)[tok * p.ldbeta + x.h]);
  return sigmoidf_rel(b);
}

__device__ __forceinline__ void prep_bar() { named_bar_sync(1, PREP_THREADS); }

__device__ __forceinline__ void prep_chunk(const ChunkParams& p, const PrepCtx& x, uint8_t* smem, int chunk, float beta_cur) {
  const int rs = chunk & 1, cs = chunk & 1;
  const int nvalid = min(C, x.len - chunk * C);
  uint8_t* raw = smem + OFF_RAW + rs * RAW_STAGE;
  uint8_t* cons = smem + OFF_CONS + cs * CS_STAGE;
  float* Gsm = reinterpret_cast<float*>(smem + OFF_G);
  float* Lsm = reinterpret_cast<float*>(smem + OFF_L);
  float* fr = reinterpret_cast<float*>(smem + OFF_FR);
  float* fer = fr + D;
  float* felr = fr + 2 * D;
  float* beta_s = reinterpret_cast<float*>(smem + OFF_BETA);
  const int lane = x.lane, pw = x.pw;

  // ---- A: gate activation and inclusive cumulative log2-decay per channel (one channel per thread)
  {
    const int ch = x.ptid;
    float run = 0.0f, r = 0.0f;
    if (p.frontend == 1) {
      const float* g = reinterpret_cast<const float*>(raw + RAW_G);
#pragma unroll
      for (int tok = 0; tok < C; tok++) {
        float a = g[tok * D + ch] * LOG2E;
        if (tok >= nvalid) a = 0.0f;
        run += a;
        Gsm[tok * D + ch] = run;
        if (tok == HALF - 1) r = run;
      }
    } else {
      const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(raw + RAW_G);
      const float c2 = p.lower_bound * LOG2E;
#pragma unroll
      for (int tok = 0; tok < C; tok++) {
        float a = c2 * sigmoidf_rel(x.eA * (__bfloat162float(g[tok * D + ch]) + x.dtb));
        if (tok >= nvalid) a = 0.0f;
        run += a;
        Gsm[tok * D + ch] = run;
        if (tok == HALF - 1) r = run;
      }
    }
    fr[ch] = r;
    fer[ch] = ex2f(r);
    felr[ch] = ex2f(run - r);
    reinterpret_cast<float*>(cons + CS_DEC)[ch] = ex2f(run);
    if (x.ptid < C) beta_s[x.ptid] = beta_cur;
  }
  prep_bar();

  // ---- B: L2 norm and the six decayed operand tiles (a warp walks 8 tokens, a lane owns 4 channels)
  {
    const float4 r4 = *reinterpret_cast<const float4*>(fr + 4 * lane);
    const float4 er4 = *reinterpret_cast<const float4*>(fer + 4 * lane);
    const float4 elr4 = *reinterpret_cast<const float4*>(felr + 4 * lane);
    const float rr[4] = {r4.x, r4.y, r4.z, r4.w};
    const float er[4] = {er4.x, er4.y, er4.z, er4.w};
    const float elr[4] = {elr4.x, elr4.y, elr4.z, elr4.w};
#pragma unroll 2
    for (int tt = 0; tt < 8; tt++) {
      const int tok = 8 * pw + tt;
      const uint2 q2 = *reinterpret_cast<const uint2*>(raw + RAW_Q + tok * 256 + lane * 8);
      const uint2 k2 = *reinterpret_cast<const uint2*>(raw + RAW_K + tok * 256 + lane * 8);
      const float qf[4] = {bf16_lo(q2.x), bf16_hi(q2.x), bf16_lo(q2.y), bf16_hi(q2.y)};
      const float kf[4] = {bf16_lo(k2.x), bf16_hi(k2.x), bf16_lo(k2.y), bf16_hi(k2.y)};
      float qinv = p.scale, kinv = 1.0f;
      if (p.frontend == 0) {
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
      float kds[4], qds[4], kis[4], kdt[4], qdt[4], krr[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float e = fminf(fmaxf(Gv[j] - rr[j], -126.0f), 126.0f);
        const float E = ex2f(e), Ei = ex2f(-e);
        const float kn = kf[j] * kinv, qn = qf[j] * qinv;
        kds[j] = kn * E; qds[j] = qn * E; kis[j] = kn * Ei;
        kdt[j] = kds[j] * er[j]; qdt[j] = qds[j] * er[j]; krr[j] = kis[j] * elr[j];
      }
      const uint32_t off = tile128_off(tok, 4 * lane);
      *reinterpret_cast<uint2*>(smem + OFF_KDS + off) = make_uint2(pack_bf16(kds[0], kds[1]), pack_bf16(kds[2], kds[3]));
      *reinterpret_cast<uint2*>(smem + OFF_QDS + off) = make_uint2(pack_bf16(qds[0], qds[1]), pack_bf16(qds[2], qds[3]));
      *reinterpret_cast<uint2*>(smem + OFF_KIS + off) = make_uint2(pack_bf16(kis[0], kis[1]), pack_bf16(kis[2], kis[3]));
      *reinterpret_cast<uint2*>(cons + CS_KD + off) = make_uint2(pack_bf16(kdt[0], kdt[1]), pack_bf16(kdt[2], kdt[3]));
      *reinterpret_cast<uint2*>(cons + CS_QD + off) = make_uint2(pack_bf16(qdt[0], qdt[1]), pack_bf16(qdt[2], qdt[3]));
      *reinterpret_cast<uint2*>(cons + CS_KR + off) = make_uint2(pack_bf16(krr[0], krr[1]), pack_bf16(krr[2], krr[3]));
    }
  }
  prep_bar();

  // ---- C: A = kd' ki'^T (warps 0,1) and M = qd' ki'^T (warps 2,3), 16 rows x 32 columns per warp
  {
    const int which = pw >> 1, rb = pw & 1;
    const uint32_t a_tile = smem_u32(smem + (which ? OFF_QDS : OFF_KDS));
    const uint32_t b_tile = smem_u32(smem + OFF_KIS);
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    const int a_row = 16 * rb + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int b_row = 8 * (lane >> 4) + (lane & 7);
#pragma unroll
    for (int kt = 0; kt < 8; kt++) {
      uint32_t a[4], b[4];
      ldmatrix_x4(a, a_tile + tile128_off(a_row, (2 * kt + (lane >> 4)) * 8));
      ldmatrix_x4(b, b_tile + tile128_off(b_row, (2 * kt + ((lane >> 3) & 1)) * 8));
      mma_bf16(acc[0], a, b[0], b[1]);
      mma_bf16(acc[1], a, b[2], b[3]);
      if (rb) {
        ldmatrix_x4(b, b_tile + tile128_off(16 + b_row, (2 * kt + ((lane >> 3) & 1)) * 8));
        mma_bf16(acc[2], a, b[0], b[1]);
        mma_bf16(acc[3], a, b[2], b[3]);
      }
    }
    const int g = lane >> 2, t = lane & 3;
    const int i0 = 16 * rb + g, i1 = i0 + 8;
    if (which == 0) {
      const float b0 = beta_s[i0], b1 = beta_s[i1];
#pragma unroll
      for (int nt = 0; nt < 4; nt++) {
        const int j = 8 * nt + 2 * t;
        Lsm[i0 * C + j] = (j < i0) ? acc[nt][0] * b0 : 0.0f;
        Lsm[i0 * C + j + 1] = (j + 1 < i0) ? acc[nt][1] * b0 : 0.0f;
        Lsm[i1 * C + j] = (j < i1) ? acc[nt][2] * b1 : 0.0f;
        Lsm[i1 * C + j + 1] = (j + 1 < i1) ? acc[nt][3] * b1 : 0.0f;
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < 4; nt++) {
        const int j = 8 * nt + 2 * t;
        const float m00 = (j <= i0) ? acc[nt][0] : 0.0f, m01 = (j + 1 <= i0) ? acc[nt][1] : 0.0f;
        const float m10 = (j <= i1) ? acc[nt][2] : 0.0f, m11 = (j + 1 <= i1) ? acc[nt][3] : 0.0f;
        *reinterpret_cast<uint32_t*>(cons + CS_MM + tile32_off(i0, j)) = pack_bf16(m00, m01);
        *reinterpret_cast<uint32_t*>(cons + CS_MM + tile32_off(i1, j)) = pack_bf16(m10, m11);
      }
    }
  }
  prep_bar();

  // ---- D: T = (I + L)^-1 by forward substitution in fp32 (lane = column), Tb = T diag(beta) as bf16
  if (pw == 0) {
    float Tc[C];
#pragma unroll
    for (int i = 0; i < C; i++) {
      float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
      for (int j = 0; j + 3 < i; j += 4) {
        const float4 l4 = *reinterpret_cast<const float4*>(Lsm + i * C + j);
        a0 = fmaf(l4.x, Tc[j], a0);
        a1 = fmaf(l4.y, Tc[j + 1], a1);
        a2 = fmaf(l4.z, Tc[j + 2], a2);
        a3 = fmaf(l4.w, Tc[j + 3], a3);
      }
#pragma unroll
      for (int j = i & ~3; j < i; j++) a0 = fmaf(Lsm[i * C + j], Tc[j], a0);
      Tc[i] = ((i == lane) ? 1.0f : 0.0f) - ((a0 + a1) + (a2 + a3));
    }
    const float bc = beta_s[lane];
#pragma unroll
    for (int i = 0; i < C; i++)
      *reinterpret_cast<__nv_bfloat16*>(cons + CS_TB + tile32_off(i, lane)) = __float2bfloat16_rn(Tc[i] * bc);
  }
}

// ------------------------------------------------------------------------------------------------ state role
__device__ __forceinline__ void state_chunk(const ChunkParams& p, const Task& task, float (&S)[16][4], uint8_t* smem,
                                            int chunk, int h, int warp, int lane) {
  const uint8_t* cons = smem + OFF_CONS + (chunk & 1) * CS_STAGE;
  const uint32_t kd_t = smem_u32(cons + CS_KD), qd_t = smem_u32(cons + CS_QD), kr_t = smem_u32(cons + CS_KR);
  const uint32_t tb_t = smem_u32(cons + CS_TB), mm_t = smem_u32(cons + CS_MM);
  const float* dec = reinterpret_cast<const float*>(cons + CS_DEC);
  const uint32_t v_t = smem_u32(smem + OFF_V + (chunk % 3) * 8192);
  const int t = lane & 3;
  const int frag_row = 8 * (lane >> 4) + (lane & 7);   // row within a 16-row pair of 8x8 matrices
  const int frag_chunk = (lane >> 3) & 1;

  float W[4][4], O[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) { W[i][j] = 0.0f; O[i][j] = 0.0f; }

  // Wt = St kd^T, Ot = St qd^T   (A = bf16(St) straight from the accumulator fragments)
#pragma unroll
  for (int kt = 0; kt < 8; kt++) {
    const uint32_t a[4] = {pack_bf16(S[2 * kt][0], S[2 * kt][1]), pack_bf16(S[2 * kt][2], S[2 * kt][3]),
                           pack_bf16(S[2 * kt + 1][0], S[2 * kt + 1][1]), pack_bf16(S[2 * kt + 1][2], S[2 * kt + 1][3])};
#pragma unroll
    for (int np = 0; np < 2; np++) {
      const uint32_t off = tile128_off(16 * np + frag_row, (2 * kt + frag_chunk) * 8);
      uint32_t b[4];
      ldmatrix_x4(b, kd_t + off);
      mma_bf16(W[2 * np], a, b[0], b[1]);
      mma_bf16(W[2 * np + 1], a, b[2], b[3]);
      ldmatrix_x4(b, qd_t + off);
      mma_bf16(O[2 * np], a, b[0], b[1]);
      mma_bf16(O[2 * np + 1], a, b[2], b[3]);
    }
  }

  // Rt = v^T - Wt  -> A fragments over the token dimension
  uint32_t ra[2][4];
#pragma unroll
  for (int np = 0; np < 2; np++) {
    uint32_t vr[4] = {0u, 0u, 0u, 0u};
    if (!(task.flags & TF_V_ZERO)) ldmatrix_x4_trans(vr, v_t + tile128_off(16 * np + frag_row, (2 * warp + frag_chunk) * 8));
    ra[np][0] = pack_bf16(bf16_lo(vr[0]) - W[2 * np][0], bf16_hi(vr[0]) - W[2 * np][1]);
    ra[np][1] = pack_bf16(bf16_lo(vr[1]) - W[2 * np][2], bf16_hi(vr[1]) - W[2 * np][3]);
    ra[np][2] = pack_bf16(bf16_lo(vr[2]) - W[2 * np + 1][0], bf16_hi(vr[2]) - W[2 * np + 1][1]);
    ra[np][3] = pack_bf16(bf16_lo(vr[3]) - W[2 * np + 1][2], bf16_hi(vr[3]) - W[2 * np + 1][3]);
  }

  // Ut = Rt Tb^T   (Tb lower triangular: the block (rows < 16, columns >= 16) is zero)
  float U[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) U[i][j] = 0.0f;
#pragma unroll
  for (int kt = 0; kt < 2; kt++) {
#pragma unroll
    for (int np = 0; np < 2; np++) {
      if (kt == 1 && np == 0) continue;
      uint32_t b[4];
      ldmatrix_x4(b, tb_t + tile32_off(16 * np + frag_row, (2 * kt + frag_chunk) * 8));
      mma_bf16(U[2 * np], ra[kt], b[0], b[1]);
      mma_bf16(U[2 * np + 1], ra[kt], b[2], b[3]);
    }
  }
  uint32_t ua[2][4];
#pragma unroll
  for (int np = 0; np < 2; np++) {
    ua[np][0] = pack_bf16(U[2 * np][0], U[2 * np][1]);
    ua[np][1] = pack_bf16(U[2 * np][2], U[2 * np][3]);
    ua[np][2] = pack_bf16(U[2 * np + 1][0], U[2 * np + 1][1]);
    ua[np][3] = pack_bf16(U[2 * np + 1][2], U[2 * np + 1][3]);
  }

  // Ot += Ut M^T
#pragma unroll
  for (int kt = 0; kt < 2; kt++) {
#pragma unroll
    for (int np = 0; np < 2; np++) {
      if (kt == 1 && np == 0) continue;
      uint32_t b[4];
      ldmatrix_x4(b, mm_t + tile32_off(16 * np + frag_row, (2 * kt + frag_chunk) * 8));
      mma_bf16(O[2 * np], ua[kt], b[0], b[1]);
      mma_bf16(O[2 * np + 1], ua[kt], b[2], b[3]);
    }
  }

  // St = St diag(2^G31) + Ut kr
#pragma unroll
  for (int nt = 0; nt < 16; nt++) {
    const float2 d2 = *reinterpret_cast<const float2*>(dec + 8 * nt + 2 * t);
    S[nt][0] *= d2.x; S[nt][1] *= d2.y; S[nt][2] *= d2.x; S[nt][3] *= d2.y;
  }
  const int kr_row = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
  for (int kt = 0; kt < 2; kt++) {
#pragma unroll
    for (int np = 0; np < 8; np++) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, kr_t + tile128_off(16 * kt + kr_row, (2 * np + (lane >> 4)) * 8));
      mma_bf16(S[2 * np], ua[kt], b[0], b[1]);
      mma_bf16(S[2 * np + 1], ua[kt], b[2], b[3]);
    }
  }

  // output rows: transpose through the warp's private slab, then 32-byte row pieces to global memory
  if (!(task.flags & TF_NO_OUT)) {
    uint8_t* slab = smem + OFF_SLAB + warp * 32 * SLAB_ROW;
    const uint32_t slab_u = smem_u32(slab);
#pragma unroll
    for (int np = 0; np < 2; np++) {
      const uint32_t r[4] = {pack_bf16(O[2 * np][0], O[2 * np][1]), pack_bf16(O[2 * np][2], O[2 * np][3]),
                             pack_bf16(O[2 * np + 1][0], O[2 * np + 1][1]), pack_bf16(O[2 * np + 1][2], O[2 * np + 1][3])};
      stmatrix_x4_trans(slab_u + (16 * np + frag_row) * SLAB_ROW + frag_chunk * 16, r);
    }
    __syncwarp();
    const int nvalid = min(C, task.len - chunk * C);
    if (lane < nvalid) {
      const uint4 lo = *reinterpret_cast<const uint4*>(slab + lane * SLAB_ROW);
      const uint4 hi = *reinterpret_cast<const uint4*>(slab + lane * SLAB_ROW + 16);
      __nv_bfloat16* o = ((task.flags & TF_OUT_AUX) ? p.out_aux : p.out) +
                         (task.t0 + (long long)chunk * C + lane) * p.ldo + (long long)h * D + 16 * warp;
      *reinterpret_cast<uint4*>(o) = lo;
      *reinterpret_cast<uint4*>(o + 8) = hi;
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(THREADS, 1) kda_chunk_fwd_kernel(const ChunkParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = p.H;
  const int rank = blockIdx.x / H, h = blockIdx.x % H;

  const int nt_word = *p.n_tasks;
  if (nt_word & NT_ZERO_FILL) {
    // rejected cu_seqlens: every sequence is empty; output rows are zero-filled so nothing is left uninitialised
    const long long rows = p.T * H;
    for (long long r = blockIdx.x; r < rows; r += gridDim.x)
      if (tid < 16) reinterpret_cast<uint4*>(p.out + (r / H) * p.ldo + (r % H) * D)[tid] = make_uint4(0, 0, 0, 0);
  }
  if (rank >= (nt_word & (NT_ZERO_FILL - 1))) return;
  const Task task = p.tasks[rank];
  const int nchunks = (task.len + C - 1) / C;

  float S[16][4];
  PrepCtx x;
  float beta_next = 0.0f;
  if (warp < STATE_WARPS) {
    load_state(S, task, h, p.key_first, warp, lane);
  } else {
    x.ptid = tid - STATE_WARPS * 32;
    x.pw = x.ptid >> 5;
    x.lane = lane;
    x.h = h;
    x.t0 = task.t0;
    x.len = task.len;
    x.eA = 0.0f;
    x.dtb = 0.0f;
    if (p.frontend == 0) {
      x.eA = __expf(p.A_log[h]);
      x.dtb = p.dt_bias[h * D + x.ptid];
    }
    if (nchunks > 0) {
      prep_issue_loads(p, x, smem, 0);
      if (x.ptid < C) beta_next = prep_load_beta(p, x, 0, x.ptid);
    }
    cp_async_commit();
  }

  for (int i = 0; i <= nchunks; i++) {
    if (warp < STATE_WARPS) {
      if (i > 0) {
        const int c = i - 1;
        if (task.ck != nullptr && p.ck_every_chunks > 0 && (c % p.ck_every_chunks) == 0) {
          const long long off = (long long)(c / p.ck_every_chunks) * p.ck_row_stride + (long long)h * STATE_ELEMS;
          if (p.ck_is_bf16) store_state_t<__nv_bfloat16>(S, reinterpret_cast<__nv_bfloat16*>(task.ck) + off, p.key_first, warp, lane);
          else store_state_t<float>(S, reinterpret_cast<float*>(task.ck) + off, p.key_first, warp, lane);
        }
        state_chunk(p, task, S, smem, c, h, warp, lane);
      }
    } else {
      if (i < nchunks) {
        const float beta_cur = beta_next;
        if (i + 1 < nchunks) {
          prep_issue_loads(p, x, smem, i + 1);
          if (x.ptid < C) beta_next = prep_load_beta(p, x, i + 1, x.ptid);
        }
        cp_async_commit();
        cp_async_wait<1>();
        prep_bar();
        prep_chunk(p, x, smem, i, beta_cur);
      }
    }
    __syncthreads();
  }

  if (warp < STATE_WARPS && task.dst != nullptr)
    store_state_t<float>(S, task.dst + (size_t)h * STATE_ELEMS, p.key_first && !(task.flags & TF_DST_VF), warp, lane);
}

cudaError_t launch_chunk_fwd(const ChunkParams& p, int n_task_cap, cudaStream_t stream) {
  static bool attr_set = false;   // per process; the attribute is per device, so set it on every device once
  static int attr_dev_mask = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set || !(attr_dev_mask & (1 << (dev & 31)))) {
    cudaError_t e = cudaFuncSetAttribute(kda_chunk_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr_set = true;
    attr_dev_mask |= 1 << (dev & 31);
  }
  const long long blocks = (long long)n_task_cap * p.H;
  if (blocks <= 0) return cudaSuccess;
  kda_chunk_fwd_kernel<<<(unsigned)blocks, THREADS, SMEM_BYTES, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace kda
