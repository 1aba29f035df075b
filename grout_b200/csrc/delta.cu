// The gated delta rule: a mixer whose memory is one matrix S [dk, dv] per head and
// sequence, updated token by token,
//
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
//
// with g in (0, 1) a decay per head and token, beta in (0, 1) a step size, k a
// unit vector and q a unit vector times dk^(-1/2).  q, k and v come out of short
// causal convolutions over time (one filter per channel, no bias, zeros before
// the sequence's start) followed by silu; the read-out o is RMS-normalised over
// dv, multiplied by a weight shared by the heads and by silu of a gate.
//
// Everything here is 32-bit whatever the activation type: the one projection
// that feeds it arrives as 32-bit sums, and only y, the o projection's input, is
// rounded.  Four kernels:
//
//   prepare  one block per token and kv head (its q and k) or run of value
//            channels: convolution (from the rows of this step and, for the first
//            tokens of a continued sequence, from the kept tail), silu, unit
//            vectors, beta, decay
//   gram     one block per group of 4 consecutive rows of a sequence and head: the
//            products k_i . k_j (i < j) and k_i . q_j (i <= j) inside the group, and
//            with them and the group's g and beta every scalar of the group that
//            does not depend on the column
//   scan     the recurrence.  The columns of S are independent recurrences, so a
//            column is held in the registers of 8 lanes (dk / 8 elements each),
//            16 columns a block, and a sequence's rows are walked in order, four
//            at a time: with c_j = g_1 .. g_j and s_0 the column before the group,
//              s_{j-1} . k_j = c_{j-1} (s_0 . k_j) + sum_{i<j} (c_{j-1} / c_i) (k_i . k_j) u_i
//              o_j = c_j (s_0 . q_j) + sum_{i<=j} (c_j / c_i) (k_i . q_j) u_i
//              s_4 = c_4 s_0 + sum_i (c_4 / c_i) k_i u_i
//            so the eight sums over dk that a group needs are taken from the column
//            as it stands, in one pass of shuffles, and what is sequential is a few
//            operations on scalars (the quotients are products of the g between, never
//            divisions).  The operands of 16 tokens at a time (their head's k and q,
//            the block's 16 values, beta, g, the group's products) reach shared memory
//            by asynchronous copies, two chunks in flight.  Groups are counted from the
//            first row a step brings, so a sequence cut elsewhere gives the same
//            result up to rounding, not bit for bit.
//   finish   one warp per (token, head): norm over dv, weight, gate; the block of a
//            sequence's first row then keeps the new tail of taps - 1 inputs
//
// Columns of the projection: q [G dk] | k [G dk] | v [H dv] | gate [H dv] | b [H] | a [H].
// A sequence's state is one row of floats: the tail [taps - 1, Cc] (Cc = the
// convolved channels q | k | v), then S as [H, dv, dk], a column's dk elements
// side by side.  Rows of slot < 0 (padding) read zeros and store nothing.
#include "attn_mma.cuh"   // the asynchronous-copy helpers

struct DeltaArgs {
  const float* proj;       // [n_tokens, C_all]
  const float* conv_w;     // [Cc, taps], the last column is the current token's
  const float* a_log;      // [H]
  const float* dt_bias;    // [H]
  const float* norm_w;     // [dv]
  const int* token_seq;    // [n_tokens]
  const int* cu_q;         // [n_seqs + 1]
  const int* slots;        // [n_seqs]
  float* state;            // [slots, state_stride]
  long long state_stride;
  float* prep;             // [n_tokens, prep_stride]: unit q | unit k | v | beta | decay | (pad to 4) |
                           //   on a group's first row: its scalars [H, 48]
  float* o;                // [n_tokens, H, dv]
  void* y;                 // [n_tokens, H dv] in the activation type
  int n_tokens, n_seqs, H, G, dk, dv, taps;
  float unit_eps, norm_eps;
  int prep_stride;         // floats between rows of prep: round4(Cc + 2 H) + 48 H
  int few_rows;            // 1: no sequence brings more than DELTA_B rows, 2: none more than one (a decode
                           //   step): the scan works out its one group's scalars itself, `gram` is not launched
};

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// One block per (token, unit): unit g < G is kv head g's q and k together, the units after that are runs of
// DELTA_PREP_V value channels; the block of unit 0 also takes beta and the decay.
#define DELTA_PREP_V 256
#define DELTA_MAX_TAPS 8     // taps fetched together; more are walked in turns

__device__ __forceinline__ float delta_conv(const DeltaArgs& a, const float* tail, int t, int r,
                                            int c, int Cc, int C_all) {
  const int taps = a.taps;
  float acc = 0.f;
  for (int j0 = 0; j0 < taps; j0 += DELTA_MAX_TAPS) {
    float x[DELTA_MAX_TAPS], w[DELTA_MAX_TAPS];
#pragma unroll
    for (int jj = 0; jj < DELTA_MAX_TAPS; ++jj) {      // all loads first: one trip to memory
      const int j = j0 + jj, rr = r - j;               // the input j tokens back
      x[jj] = 0.f, w[jj] = 0.f;
      if (j < taps) {
        w[jj] = a.conv_w[(size_t)c * taps + taps - 1 - j];
        if (rr >= 0) x[jj] = a.proj[(size_t)(t - j) * C_all + c];
        else if (tail) x[jj] = tail[(size_t)(taps - 1 + rr) * Cc + c];
      }
    }
#pragma unroll
    for (int jj = 0; jj < DELTA_MAX_TAPS; ++jj) acc = fmaf(w[jj], x[jj], acc);
  }
  return silu_f(acc);
}

__global__ void __launch_bounds__(256) delta_prepare_kernel(const DeltaArgs a) {
  extern __shared__ float row[];   // [2 dk]: a kv head's q and k after the convolution
  __shared__ float scratch[32];
  pdl_launch_dependents_if_small();
  const int t = blockIdx.x, unit = blockIdx.y, tid = threadIdx.x;
  const int H = a.H, G = a.G, dk = a.dk, dv = a.dv;
  const int Cc = 2 * G * dk + H * dv, C_all = Cc + H * dv + 2 * H, P = a.prep_stride;
  const int seq = a.token_seq[t];
  const int slot = a.slots[seq];
  const int r = t - a.cu_q[seq];                 // the token's place among its sequence's rows
  const float* tail = slot >= 0 ? a.state + (size_t)slot * a.state_stride : nullptr;
  float* out = a.prep + (size_t)t * P;
  pdl_wait();
  if (unit >= G) {                               // value channels: convolution and silu
    const int c = 2 * G * dk + (unit - G) * DELTA_PREP_V + tid;
    if (tid < DELTA_PREP_V && c < Cc) out[c] = delta_conv(a, tail, t, r, c, Cc, C_all);
    return;
  }
  float sq = 0.f, sk = 0.f;
  for (int i = tid; i < 2 * dk; i += blockDim.x) {
    const int c = i < dk ? unit * dk + i : (G + unit) * dk + (i - dk);
    const float v = delta_conv(a, tail, t, r, c, Cc, C_all);
    row[i] = v;
    if (i < dk) sq += v * v; else sk += v * v;
  }
  sq = block_sum(sq, scratch);
  sk = block_sum(sk, scratch);
  const float iq = 1.0f / sqrtf(sq + a.unit_eps) * (1.0f / sqrtf((float)dk));
  const float ik = 1.0f / sqrtf(sk + a.unit_eps);
  for (int d = tid; d < dk; d += blockDim.x) {
    out[unit * dk + d] = row[d] * iq;
    out[(G + unit) * dk + d] = row[dk + d] * ik;
  }
  if (unit == 0) {
    for (int h = tid; h < H; h += blockDim.x) {
      const float b = a.proj[(size_t)t * C_all + Cc + H * dv + h];
      const float al = a.proj[(size_t)t * C_all + Cc + H * dv + H + h];
      out[Cc + h] = 1.0f / (1.0f + expf(-b));
      out[Cc + H + h] = expf(-expf(a.a_log[h]) * softplus_f(al + a.dt_bias[h]));
    }
  }
  pdl_launch_dependents_if_large();
}

// The new tail of a sequence: the last taps - 1 inputs of its convolutions.  Entry s
// holds the input at n - (taps - 1) + s rows from the step's first; an entry that stays
// is read (at n + s > s) before anything at or above it is written.
__device__ __forceinline__ void delta_keep_tail(const DeltaArgs& a, int seq) {
  const int slot = a.slots[seq];
  const int row0 = a.cu_q[seq], n = a.cu_q[seq + 1] - row0;
  if (slot < 0 || n <= 0) return;
  const int taps = a.taps;
  const int Cc = 2 * a.G * a.dk + a.H * a.dv, C_all = Cc + a.H * a.dv + 2 * a.H;
  float* tail = a.state + (size_t)slot * a.state_stride;
  // the blocks of the row (blockIdx.y) share the channels; up to eight entries are read
  // together before any of them is written
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < Cc; c += gridDim.y * blockDim.x) {
    for (int s0 = 0; s0 < taps - 1; s0 += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int s = s0 + u, rr = n - (taps - 1) + s;
        v[u] = 0.f;
        if (s < taps - 1)
          v[u] = rr >= 0 ? a.proj[(size_t)(row0 + rr) * C_all + c] : tail[(size_t)(taps - 1 + rr) * Cc + c];
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (s0 + u < taps - 1) tail[(size_t)(s0 + u) * Cc + c] = v[u];
    }
  }
}

#define DELTA_LANES 8       // lanes that share a column of S
#define DELTA_COLS 16       // columns of S per block
#define DELTA_TT 16         // tokens whose operands are staged together
#define DELTA_B 4           // rows of a group

__host__ __device__ __forceinline__ int delta_gram_offset(int Cc, int H) { return (Cc + 2 * H + 3) / 4 * 4; }

// The scalars of a group of DELTA_B rows and one head that do not depend on the column
// (c_j = g_1 .. g_j, c_0 = 1; quotients c_j / c_i are products of the g between):
//   [0, 4)   A_j  = beta_j g_j c_{j-1}                       u_j = beta_j v_j - A_j (s_0 . k_j)
//   [4, 20)  C_ij = beta_j g_j (c_{j-1} / c_i) (k_i . k_j)          - sum_{i<j} C_ij u_i
//   [20, 24) c_j                                              o_j = c_j (s_0 . q_j)
//   [24, 40) D_ij = (c_j / c_i) (k_i . q_j)                         + sum_{i<=j} D_ij u_i
//   [40, 44) E_i  = c_4 / c_i                                 s_4 = c_4 s_0 + sum_i E_i u_i k_i
//   [44, 48) beta_j
// Rows beyond the sequence's end are neutral (beta 0, g 1, products 0).
#define DELTA_COEF 48
// Where the pieces lie for groups of B rows (B = 4: the table above); the whole is filled up
// to a multiple of four floats.
template <int B> struct DeltaCoef {
  static constexpr int A = 0, C = B, CUM = B + B * B, D = 2 * B + B * B, E = 2 * B + 2 * B * B,
                       BETA = 3 * B + 2 * B * B, SIZE = (4 * B + 2 * B * B + 3) / 4 * 4;
};
static_assert(DeltaCoef<DELTA_B>::SIZE == DELTA_COEF, "the scalars of a group of four rows are 48 floats");

template <int B>
__device__ __forceinline__ void delta_group_scalars(float* out, const float* dots,
                                                    const float (&beta)[B], const float (&g)[B]) {
  using L = DeltaCoef<B>;
  float quot[B][B], cum[B + 1];
  cum[0] = 1.f;
  for (int j = 0; j < B; ++j) {
    cum[j + 1] = cum[j] * g[j];
    quot[j][j] = 1.f;
    for (int i = 0; i < j; ++i) quot[i][j] = quot[i][j - 1] * g[j];
  }
  for (int j = 0; j < B; ++j) {
    out[L::A + j] = beta[j] * g[j] * cum[j];
    out[L::CUM + j] = cum[j + 1];
    out[L::E + j] = quot[j][B - 1];
    out[L::BETA + j] = beta[j];
    for (int i = 0; i < B; ++i) {
      out[L::C + i * B + j] = i < j ? beta[j] * g[j] * quot[i][j - 1] * dots[i * B + j] : 0.f;
      out[L::D + i * B + j] = i <= j ? quot[i][j] * dots[B * B + i * B + j] : 0.f;
    }
  }
}

__global__ void __launch_bounds__(128) delta_gram_kernel(const DeltaArgs a) {
  __shared__ float dots[2 * DELTA_B * DELTA_B];
  pdl_launch_dependents_if_small();
  constexpr int B = DELTA_B;
  const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.G, H = a.H, dk = a.dk, P = a.prep_stride;
  const int Cc = 2 * G * dk + H * a.dv, kvh = h / (H / G);
  const int seq = a.token_seq[t];
  const int row0 = a.cu_q[seq], r = t - row0;
  if (r % B) return;
  const int nb = min(B, a.cu_q[seq + 1] - t);
  pdl_wait();
  for (int e = warp; e < 2 * B * B; e += 4) {       // e < 16: k_i . k_j, else k_i . q_j
    const int with_q = e / (B * B), i = (e % (B * B)) / B, j = e % B;
    float acc = 0.f;
    if (i < nb && j < nb && (with_q ? i <= j : i < j)) {
      const float* ki = a.prep + (size_t)(t + i) * P + (G + kvh) * dk;
      const float* xj = a.prep + (size_t)(t + j) * P + (with_q ? kvh : G + kvh) * dk;
      for (int d = lane; d < dk; d += 32) acc = fmaf(ki[d], xj[d], acc);
      acc = warp_sum(acc);
    }
    if (lane == 0) dots[e] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float beta[B], g[B];
    for (int j = 0; j < B; ++j) {
      beta[j] = j < nb ? a.prep[(size_t)(t + j) * P + Cc + h] : 0.f;
      g[j] = j < nb ? a.prep[(size_t)(t + j) * P + Cc + H + h] : 1.f;
    }
    delta_group_scalars<DELTA_B>(a.prep + (size_t)t * P + delta_gram_offset(Cc, H) + h * DELTA_COEF, dots, beta, g);
  }
  pdl_launch_dependents_if_large();
}

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem));
}

// R floats of a column per lane, in pieces of four: piece i of lane l holds the
// elements (i * 8 + l) * 4 .. + 3, so that the lanes of a column read contiguous
// bytes of shared memory, and of the state, at a time.
// B = 4 rows a turn; B = 1 for a step in which every sequence brings one row (a decode step):
// one staged row, one group, far fewer registers, so that more of its many short blocks fit an SM.
template <int R, int B>
__global__ void __launch_bounds__(DELTA_LANES * DELTA_COLS) delta_scan_kernel(const DeltaArgs a) {
  extern __shared__ __align__(16) float sm[];
  using L = DeltaCoef<B>;
  constexpr int TT = B == 1 ? 1 : DELTA_TT;            // rows of a stage
  constexpr int DKP = DELTA_LANES * R;                       // dk filled up with zeros
  constexpr int GRAM = L::SIZE;
  // q | k | v | the groups' scalars
  constexpr int STAGE = TT * (2 * DKP + DELTA_COLS) + (TT / B) * GRAM;
  pdl_launch_dependents_if_small();
  const int seq = blockIdx.z, h = blockIdx.y, tid = threadIdx.x;
  const int col0 = blockIdx.x * DELTA_COLS;
  const int col = col0 + tid / DELTA_LANES, l = tid % DELTA_LANES;
  const int H = a.H, G = a.G, dk = a.dk, dv = a.dv;
  const int Cc = 2 * G * dk + H * dv, P = a.prep_stride;
  const int gram_off = delta_gram_offset(Cc, H);
  const int kvh = h / (H / G);
  const bool active = col < dv;
  if (dk < DKP)   // what no copy writes stays zero (a step of few rows has one stage only)
    for (int i = tid; i < (a.few_rows ? 1 : 2) * STAGE; i += blockDim.x) sm[i] = 0.f;
  pdl_wait();
  const int row0 = a.cu_q[seq], n = a.cu_q[seq + 1] - row0;
  if (n <= 0) return;
  __syncthreads();
  const int slot = a.slots[seq];
  float* sp = slot >= 0 && active
                  ? a.state + (size_t)slot * a.state_stride + (size_t)(a.taps - 1) * Cc +
                        ((size_t)h * dv + col) * dk
                  : nullptr;
  const bool wide = (dk & 3) == 0;     // 16-byte copies; prep rows are 16-byte aligned
  const bool wide_state = wide && sp && (((uintptr_t)sp) & 15) == 0;
  float S[R];
#pragma unroll
  for (int i = 0; i < R / 4; ++i) {
    const int e = (i * DELTA_LANES + l) * 4;
    if (wide_state) {
      const float4 x = e < dk ? *reinterpret_cast<const float4*>(sp + e) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[4 * i] = x.x, S[4 * i + 1] = x.y, S[4 * i + 2] = x.z, S[4 * i + 3] = x.w;
    } else {
#pragma unroll
      for (int x = 0; x < 4; ++x) S[4 * i + x] = sp && e + x < dk ? sp[e + x] : 0.f;
    }
  }
  const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  auto stage_in = [&](int chunk, int st) {
    float* base = sm + st * STAGE;
    float* vs = base + 2 * TT * DKP;
    float* gr = vs + TT * DELTA_COLS;
    const int t0 = row0 + chunk * TT;
    const int nt = min(TT, row0 + n - t0);
    for (int tt = warp; tt < nt; tt += nwarps) {          // a warp per token: its q, its k, its values
      const float* src = a.prep + (size_t)(t0 + tt) * P;
      if (wide) {
        for (int pc = lane; pc < dk / 4; pc += 32) {
          cp_async16(base + tt * DKP + pc * 4, src + kvh * dk + pc * 4, true);
          cp_async16(base + (TT + tt) * DKP + pc * 4, src + (G + kvh) * dk + pc * 4, true);
        }
      } else {
        for (int d = lane; d < dk; d += 32) {
          cp_async4(base + tt * DKP + d, src + kvh * dk + d);
          cp_async4(base + (TT + tt) * DKP + d, src + (G + kvh) * dk + d);
        }
      }
      if (lane < DELTA_COLS && col0 + lane < dv)
        cp_async4(vs + tt * DELTA_COLS + lane, src + 2 * G * dk + h * dv + col0 + lane);
    }
    if (!a.few_rows)
      for (int gi = warp; gi * B < nt; gi += nwarps)      // a warp per group: its scalars
        for (int e = lane; e < GRAM / 4; e += 32)
          cp_async16(gr + gi * GRAM + e * 4, a.prep + (size_t)(t0 + gi * B) * P + gram_off + h * GRAM + e * 4, true);
    cp_async_commit();
    const int fill = ((nt + B - 1) / B) * B - nt;   // the sequence ends inside a group: its other rows are zeros
    if (fill > 0) {
      for (int i = tid; i < fill * DKP; i += blockDim.x) {
        base[nt * DKP + i] = 0.f;
        base[(TT + nt) * DKP + i] = 0.f;
      }
      for (int i = tid; i < fill * DELTA_COLS; i += blockDim.x) vs[nt * DELTA_COLS + i] = 0.f;
    }
  };
  const int n_chunks = (n + TT - 1) / TT;
  float beta_f[B], g_f[B];      // a step of few rows: the one group's beta and g, asked for early
#pragma unroll
  for (int j = 0; j < B; ++j) {
    beta_f[j] = 0.f, g_f[j] = 1.f;
    if (a.few_rows && tid == 0 && j < n) {
      beta_f[j] = a.prep[(size_t)(row0 + j) * P + Cc + h];
      g_f[j] = a.prep[(size_t)(row0 + j) * P + Cc + H + h];
    }
  }
  stage_in(0, 0);
  for (int c = 0; c < n_chunks; ++c) {
    const int st = c & 1;
    if (c + 1 < n_chunks) {
      stage_in(c + 1, st ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* base = sm + st * STAGE;
    const float* vs = base + 2 * TT * DKP;
    const float* gr = vs + TT * DELTA_COLS;
    const int t0 = row0 + c * TT;
    const int nt = min(TT, row0 + n - t0);
    if (a.few_rows) {       // the one group's products from the staged rows, then its scalars
      __shared__ float dots[2 * B * B];
      for (int e = warp; e < 2 * B * B; e += nwarps) {
        const int with_q = e / (B * B), i = (e % (B * B)) / B, j = e % B;
        float acc = 0.f;
        if (i < nt && j < nt && (with_q ? i <= j : i < j)) {
          const float* ki = base + (TT + i) * DKP;
          const float* xj = base + (with_q ? j : TT + j) * DKP;
          for (int d = lane; d < dk; d += 32) acc = fmaf(ki[d], xj[d], acc);
          acc = warp_sum(acc);
        }
        if (lane == 0) dots[e] = acc;
      }
      __syncthreads();
      if (tid == 0)
        delta_group_scalars<B>(sm + st * STAGE + 2 * TT * DKP + TT * DELTA_COLS, dots, beta_f, g_f);
      __syncthreads();
    }
    for (int g0 = 0; g0 < nt; g0 += B) {
      float k[B][R], sk[B], sq[B];
#pragma unroll
      for (int j = 0; j < B; ++j) {
        const float4* qp = reinterpret_cast<const float4*>(base + (g0 + j) * DKP) + l;
        const float4* kp = reinterpret_cast<const float4*>(base + (TT + g0 + j) * DKP) + l;
        float d1 = 0.f, d2 = 0.f;
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
          const float4 kk = kp[i * DELTA_LANES], qq = qp[i * DELTA_LANES];
          k[j][4 * i] = kk.x, k[j][4 * i + 1] = kk.y, k[j][4 * i + 2] = kk.z, k[j][4 * i + 3] = kk.w;
          d1 = fmaf(S[4 * i], kk.x, d1), d1 = fmaf(S[4 * i + 1], kk.y, d1);
          d1 = fmaf(S[4 * i + 2], kk.z, d1), d1 = fmaf(S[4 * i + 3], kk.w, d1);
          d2 = fmaf(S[4 * i], qq.x, d2), d2 = fmaf(S[4 * i + 1], qq.y, d2);
          d2 = fmaf(S[4 * i + 2], qq.z, d2), d2 = fmaf(S[4 * i + 3], qq.w, d2);
        }
        sk[j] = d1, sq[j] = d2;
      }
#pragma unroll
      for (int m = 1; m < DELTA_LANES; m <<= 1)
#pragma unroll
        for (int j = 0; j < B; ++j) {
          sk[j] += __shfl_xor_sync(0xffffffffu, sk[j], m);
          sq[j] += __shfl_xor_sync(0xffffffffu, sq[j], m);
        }
      // what is left of the group's scalars depends on the column: every lane computes the same
      const float4* cf = reinterpret_cast<const float4*>(gr + (g0 / B) * GRAM);
      float co[GRAM];
#pragma unroll
      for (int i = 0; i < GRAM / 4; ++i) {
        const float4 x = cf[i];
        co[4 * i] = x.x, co[4 * i + 1] = x.y, co[4 * i + 2] = x.z, co[4 * i + 3] = x.w;
      }
      float u[B], w[B];
#pragma unroll
      for (int j = 0; j < B; ++j) {
        const float v = vs[(g0 + j) * DELTA_COLS + (tid / DELTA_LANES)];
        float uj = fmaf(co[L::BETA + j], v, -co[L::A + j] * sk[j]);
#pragma unroll
        for (int i = 0; i < j; ++i) uj = fmaf(-co[L::C + i * B + j], u[i], uj);
        u[j] = uj;
        float o = co[L::CUM + j] * sq[j];
#pragma unroll
        for (int i = 0; i <= j; ++i) o = fmaf(co[L::D + i * B + j], u[i], o);
        if (l == 0 && active && g0 + j < nt) a.o[((size_t)(t0 + g0 + j) * H + h) * dv + col] = o;
      }
#pragma unroll
      for (int i = 0; i < B; ++i) w[i] = co[L::E + i] * u[i];
      const float cum = co[L::CUM + B - 1];
#pragma unroll
      for (int x = 0; x < R; ++x) {
        float sx = cum * S[x];
#pragma unroll
        for (int i = 0; i < B; ++i) sx = fmaf(k[i][x], w[i], sx);
        S[x] = sx;
      }
    }
    __syncthreads();   // the stage is refilled by the next turn's copies
  }
  pdl_launch_dependents_if_large();
  if (sp) {
#pragma unroll
    for (int i = 0; i < R / 4; ++i) {
      const int e = (i * DELTA_LANES + l) * 4;
      if (wide_state) {
        if (e < dk) *reinterpret_cast<float4*>(sp + e) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
      } else {
#pragma unroll
        for (int x = 0; x < 4; ++x)
          if (e + x < dk) sp[e + x] = S[4 * i + x];
      }
    }
  }
}

template <typename T>
__global__ void delta_finish_kernel(const DeltaArgs a) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int H = a.H, dv = a.dv;
  const int Cc = 2 * a.G * a.dk + H * dv, C_all = Cc + H * dv + 2 * H;
  for (int h = blockIdx.y * nwarps + warp; h < H; h += gridDim.y * nwarps) {
    const float* o = a.o + ((size_t)t * H + h) * dv;
    const float* gate = a.proj + (size_t)t * C_all + Cc + h * dv;
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) ss += o[j] * o[j];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + a.norm_eps);
    T* y = (T*)a.y + ((size_t)t * H + h) * dv;
    for (int j = lane; j < dv; j += 32) y[j] = from_f32<T>(o[j] * inv * a.norm_w[j] * silu_f(gate[j]));
  }
  // the block of a sequence's first row also keeps the convolutions' tail (every reader
  // of the old one, the prepare kernel, has finished)
  if (a.taps > 1) {
    const int seq = a.token_seq[t];
    if (t == a.cu_q[seq]) delta_keep_tail(a, seq);
  }
  pdl_launch_dependents_if_large();
}

template <int R, int B>
static int scan_launch_b(const DeltaArgs& a, cudaStream_t s) {
  const dim3 grid((a.dv + DELTA_COLS - 1) / DELTA_COLS, a.H, a.n_seqs), block(DELTA_LANES * DELTA_COLS);
  constexpr int TT = B == 1 ? 1 : DELTA_TT;
  const size_t smem = (size_t)(a.few_rows ? 1 : 2) * (TT * (2 * DELTA_LANES * R + DELTA_COLS) +
                                                      (TT / B) * DeltaCoef<B>::SIZE) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t ce = cudaFuncSetAttribute(delta_scan_kernel<R, B>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
  }
  return gb_launch(delta_scan_kernel<R, B>, grid, block, smem, s, a);
}

template <int R>
static int scan_launch(const DeltaArgs& a, cudaStream_t s) {
  return a.few_rows == 2 ? scan_launch_b<R, 1>(a, s) : scan_launch_b<R, DELTA_B>(a, s);
}

static int delta_check(const DeltaArgs& a) {
  if (a.n_tokens < 0 || a.n_seqs <= 0 || a.H <= 0 || a.G <= 0 || a.H % a.G || a.dk <= 0 ||
      a.dv <= 0 || a.taps <= 0 || !a.proj || !a.state || !a.prep || !a.o || !a.y)
    return GB_ERR_BAD_ARG;
  if (a.dk > 32 * DELTA_LANES) return GB_ERR_UNSUPPORTED;
  const int Cc = 2 * a.G * a.dk + a.H * a.dv;
  if (a.prep_stride != delta_gram_offset(Cc, a.H) + DELTA_COEF * a.H ||
      (((uintptr_t)a.prep) & 15))
    return GB_ERR_BAD_ARG;
  return 0;
}

template <typename T>
static int delta_forward(const DeltaArgs& a, cudaStream_t s) {
  int e = delta_check(a);
  if (e) return e;
  if (a.n_tokens == 0) return 0;
  const int units = a.G + (a.H * a.dv + DELTA_PREP_V - 1) / DELTA_PREP_V;
  e = gb_launch(delta_prepare_kernel, dim3(a.n_tokens, units), dim3(256),
                (size_t)2 * a.dk * sizeof(float), s, a);
  if (e) return e;
  if (!a.few_rows) {
    e = gb_launch(delta_gram_kernel, dim3(a.n_tokens, a.H), dim3(128), 0, s, a);
    if (e) return e;
  }
  const int per_lane = (a.dk + DELTA_LANES - 1) / DELTA_LANES;
  if (per_lane <= 4) e = scan_launch<4>(a, s);
  else if (per_lane <= 8) e = scan_launch<8>(a, s);
  else if (per_lane <= 12) e = scan_launch<12>(a, s);
  else if (per_lane <= 16) e = scan_launch<16>(a, s);
  else if (per_lane <= 24) e = scan_launch<24>(a, s);
  else e = scan_launch<32>(a, s);
  if (e) return e;
  const int warps = a.H < 8 ? a.H : 8;
  int rows_y = (a.H + warps - 1) / warps;            // blocks of a row: enough for its heads, and
  const int Cc = 2 * a.G * a.dk + a.H * a.dv;        //   for the tail's channels four to a thread
  const int for_tail = a.taps > 1 ? (Cc + warps * 32 * 4 - 1) / (warps * 32 * 4) : 1;
  if (for_tail > rows_y) rows_y = for_tail < 64 ? for_tail : 64;
  return gb_launch(delta_finish_kernel<T>, dim3(a.n_tokens, rows_y), dim3(warps * 32), 0, s, a);
}

// Four launches: prepare, gram (not for a step of few rows a sequence), scan, finish.
GB_EXPORT int gb_delta_forward_f32(const DeltaArgs* a, cudaStream_t s) { return delta_forward<float>(*a, s); }
GB_EXPORT int gb_delta_forward_bf16(const DeltaArgs* a, cudaStream_t s) { return delta_forward<bf16>(*a, s); }
