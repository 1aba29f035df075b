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
//   prepare  one block per token: convolution (from the rows of this step and,
//            for the first tokens of a continued sequence, from the kept tail),
//            silu, unit vectors, beta, decay
//   keep     one block per sequence: the new tail of taps - 1 inputs
//   scan     the recurrence.  The columns of S are independent recurrences, so a
//            column is held in the registers of 8 lanes (dk / 8 elements each),
//            16 columns a block, and a sequence's rows are walked in order.  A
//            token's operands (its head's k and q, the block's 16 values, beta, g)
//            reach shared memory 16 tokens at a time by asynchronous copies, two
//            chunks in flight.  Per token both S^T k and S^T q are taken from the
//            state as it stands, in one round of shuffles, and the read-out follows
//            from them: o = g S^T q + u (k . q), since S' = g S + k u^T; the update
//            of S is then off the path to the next token's sums.  A token's result
//            does not depend on how the sequence was cut into steps: the order of
//            operations is the same.
//   finish   one warp per (token, head): norm over dv, weight, gate
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
  float* prep;             // [n_tokens, prep_stride]: unit q | unit k | v | beta | decay | k . q [G]
  float* o;                // [n_tokens, H, dv]
  void* y;                 // [n_tokens, H dv] in the activation type
  int n_tokens, n_seqs, H, G, dk, dv, taps;
  float unit_eps, norm_eps;
  int prep_stride;         // floats between rows of prep: at least Cc + 2 H + G, a multiple of 4
};

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__global__ void delta_prepare_kernel(const DeltaArgs a) {
  extern __shared__ float row[];   // [Cc]
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int H = a.H, G = a.G, dk = a.dk, dv = a.dv, taps = a.taps;
  const int Cc = 2 * G * dk + H * dv, C_all = Cc + H * dv + 2 * H, P = a.prep_stride;
  const int seq = a.token_seq[t];
  const int slot = a.slots[seq];
  const int r = t - a.cu_q[seq];                 // the token's place among its sequence's rows
  const float* tail = slot >= 0 ? a.state + (size_t)slot * a.state_stride : nullptr;
  for (int c = tid; c < Cc; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {             // the input j tokens back
      const int rr = r - j;
      float x;
      if (rr >= 0) x = a.proj[(size_t)(t - j) * C_all + c];
      else x = tail ? tail[(size_t)(taps - 1 + rr) * Cc + c] : 0.f;
      acc = fmaf(a.conv_w[(size_t)c * taps + taps - 1 - j], x, acc);
    }
    row[c] = silu_f(acc);
  }
  __syncthreads();
  pdl_launch_dependents_if_large();
  float* out = a.prep + (size_t)t * P;
  const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  const float mul = 1.0f / sqrtf((float)dk);
  for (int head = warp; head < G; head += nwarps) {     // a kv head's q and k, and their product
    const float* xq = row + head * dk;
    const float* xk = row + (G + head) * dk;
    float sq = 0.f, sk = 0.f;
    for (int d = lane; d < dk; d += 32) sq += xq[d] * xq[d], sk += xk[d] * xk[d];
    sq = warp_sum(sq), sk = warp_sum(sk);
    const float iq = 1.0f / sqrtf(sq + a.unit_eps), ik = 1.0f / sqrtf(sk + a.unit_eps);
    float kq = 0.f;
    for (int d = lane; d < dk; d += 32) {
      const float qv = xq[d] * iq * mul, kv = xk[d] * ik;
      out[head * dk + d] = qv;
      out[(G + head) * dk + d] = kv;
      kq = fmaf(qv, kv, kq);
    }
    kq = warp_sum(kq);
    if (lane == 0) out[Cc + 2 * H + head] = kq;
  }
  for (int c = 2 * G * dk + tid; c < Cc; c += blockDim.x) out[c] = row[c];
  for (int h = tid; h < H; h += blockDim.x) {
    const float b = a.proj[(size_t)t * C_all + Cc + H * dv + h];
    const float al = a.proj[(size_t)t * C_all + Cc + H * dv + H + h];
    out[Cc + h] = 1.0f / (1.0f + expf(-b));
    out[Cc + H + h] = expf(-expf(a.a_log[h]) * softplus_f(al + a.dt_bias[h]));
  }
}

__global__ void delta_keep_kernel(const DeltaArgs a) {
  pdl_wait();
  const int seq = blockIdx.x;
  const int slot = a.slots[seq];
  const int row0 = a.cu_q[seq], n = a.cu_q[seq + 1] - row0;
  if (slot < 0 || n <= 0) return;
  const int taps = a.taps;
  const int Cc = 2 * a.G * a.dk + a.H * a.dv, C_all = Cc + a.H * a.dv + 2 * a.H;
  float* tail = a.state + (size_t)slot * a.state_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < Cc; c += gridDim.y * blockDim.x) {
    // entry s holds the input at n - (taps - 1) + s rows from the step's first; an
    // entry that stays is read (at n + s > s) before anything at or above it is written
    for (int s = 0; s < taps - 1; ++s) {
      const int rr = n - (taps - 1) + s;
      tail[(size_t)s * Cc + c] = rr >= 0 ? a.proj[(size_t)(row0 + rr) * C_all + c]
                                         : tail[(size_t)(taps - 1 + rr) * Cc + c];
    }
  }
}

#define DELTA_LANES 8       // lanes that share a column of S
#define DELTA_COLS 16       // columns of S per block
#define DELTA_TT 16         // tokens whose operands are staged together

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem));
}

// R floats of a column per lane, in pieces of four: piece i of lane l holds the
// elements (i * 8 + l) * 4 .. + 3, so that the eight lanes of a column read 128
// contiguous bytes of shared memory, and of the state, at a time.
template <int R>
__global__ void __launch_bounds__(DELTA_LANES * DELTA_COLS) delta_scan_kernel(const DeltaArgs a) {
  extern __shared__ __align__(16) float sm[];
  constexpr int DKP = DELTA_LANES * R;                       // dk filled up with zeros
  constexpr int STAGE = DELTA_TT * (2 * DKP + DELTA_COLS + 4);   // q | k | v | beta, g, k.q, -
  pdl_launch_dependents_if_small();
  const int seq = blockIdx.z, h = blockIdx.y, tid = threadIdx.x;
  const int col0 = blockIdx.x * DELTA_COLS;
  const int col = col0 + tid / DELTA_LANES, l = tid % DELTA_LANES;
  const int H = a.H, G = a.G, dk = a.dk, dv = a.dv;
  const int Cc = 2 * G * dk + H * dv, P = a.prep_stride;
  const int kvh = h / (H / G);
  const bool active = col < dv;
  if (dk < DKP)
    for (int i = tid; i < 2 * STAGE; i += blockDim.x) sm[i] = 0.f;   // what no copy writes stays zero
  pdl_wait();
  const int row0 = a.cu_q[seq], n = a.cu_q[seq + 1] - row0;
  if (n <= 0) return;
  __syncthreads();
  const int slot = a.slots[seq];
  float* sp = slot >= 0 && active
                  ? a.state + (size_t)slot * a.state_stride + (size_t)(a.taps - 1) * Cc +
                        ((size_t)h * dv + col) * dk
                  : nullptr;
  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int e = ((i >> 2) * DELTA_LANES + l) * 4 + (i & 3);
    S[i] = sp && e < dk ? sp[e] : 0.f;
  }
  const bool wide = (dk & 3) == 0;     // 16-byte copies; prep rows are 16-byte aligned
  auto stage_in = [&](int chunk, int st) {
    float* base = sm + st * STAGE;
    const int t0 = row0 + chunk * DELTA_TT;
    const int nt = min(DELTA_TT, row0 + n - t0);
    if (wide) {
      const int per = dk >> 2;                              // pieces of a token's q (or k)
      for (int i = tid; i < nt * 2 * per; i += blockDim.x) {
        const int tt = i / (2 * per), r = i % (2 * per), which = r / per, pc = r % per;
        const float* src = a.prep + (size_t)(t0 + tt) * P + (which * G + kvh) * dk + pc * 4;
        cp_async16(base + (which * DELTA_TT + tt) * DKP + pc * 4, src, true);
      }
    } else {
      for (int i = tid; i < nt * 2 * dk; i += blockDim.x) {
        const int tt = i / (2 * dk), r = i % (2 * dk), which = r / dk, d = r % dk;
        cp_async4(base + (which * DELTA_TT + tt) * DKP + d,
                  a.prep + (size_t)(t0 + tt) * P + (which * G + kvh) * dk + d);
      }
    }
    float* vs = base + 2 * DELTA_TT * DKP;
    float* sc = vs + DELTA_TT * DELTA_COLS;
    for (int i = tid; i < nt * DELTA_COLS; i += blockDim.x) {
      const int tt = i / DELTA_COLS, c = i % DELTA_COLS;
      if (col0 + c < dv) cp_async4(vs + i, a.prep + (size_t)(t0 + tt) * P + 2 * G * dk + h * dv + col0 + c);
    }
    for (int i = tid; i < nt * 3; i += blockDim.x) {
      const int tt = i / 3, w = i % 3;
      const int off = w == 0 ? Cc + h : (w == 1 ? Cc + H + h : Cc + 2 * H + kvh);
      cp_async4(sc + tt * 4 + w, a.prep + (size_t)(t0 + tt) * P + off);
    }
    cp_async_commit();
  };
  const int n_chunks = (n + DELTA_TT - 1) / DELTA_TT;
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
    const float* vs = base + 2 * DELTA_TT * DKP;
    const float* sc = vs + DELTA_TT * DELTA_COLS;
    const int t0 = row0 + c * DELTA_TT;
    const int nt = min(DELTA_TT, row0 + n - t0);
    for (int tt = 0; tt < nt; ++tt) {
      const float4* qp = reinterpret_cast<const float4*>(base + tt * DKP) + l;
      const float4* kp = reinterpret_cast<const float4*>(base + (DELTA_TT + tt) * DKP) + l;
      float k[R];
      float d1[4] = {0.f, 0.f, 0.f, 0.f}, d2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < R / 4; ++i) {
        const float4 kk = kp[i * DELTA_LANES], qq = qp[i * DELTA_LANES];
        k[4 * i] = kk.x, k[4 * i + 1] = kk.y, k[4 * i + 2] = kk.z, k[4 * i + 3] = kk.w;
        d1[0] = fmaf(S[4 * i], kk.x, d1[0]), d1[1] = fmaf(S[4 * i + 1], kk.y, d1[1]);
        d1[2] = fmaf(S[4 * i + 2], kk.z, d1[2]), d1[3] = fmaf(S[4 * i + 3], kk.w, d1[3]);
        d2[0] = fmaf(S[4 * i], qq.x, d2[0]), d2[1] = fmaf(S[4 * i + 1], qq.y, d2[1]);
        d2[2] = fmaf(S[4 * i + 2], qq.z, d2[2]), d2[3] = fmaf(S[4 * i + 3], qq.w, d2[3]);
      }
      float sk = (d1[0] + d1[1]) + (d1[2] + d1[3]), sq = (d2[0] + d2[1]) + (d2[2] + d2[3]);
#pragma unroll
      for (int m = 1; m < DELTA_LANES; m <<= 1) {
        sk += __shfl_xor_sync(0xffffffffu, sk, m);
        sq += __shfl_xor_sync(0xffffffffu, sq, m);
      }
      const float beta = sc[tt * 4], g = sc[tt * 4 + 1], kq = sc[tt * 4 + 2];
      const float v = vs[tt * DELTA_COLS + (tid / DELTA_LANES)];
      const float u = beta * (v - g * sk);
#pragma unroll
      for (int i = 0; i < R; ++i) S[i] = fmaf(k[i], u, g * S[i]);
      if (l == 0 && active) a.o[((size_t)(t0 + tt) * H + h) * dv + col] = fmaf(u, kq, g * sq);
    }
    __syncthreads();   // the stage is refilled by the next turn's copies
  }
  pdl_launch_dependents_if_large();
  if (sp) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int e = ((i >> 2) * DELTA_LANES + l) * 4 + (i & 3);
      if (e < dk) sp[e] = S[i];
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
  pdl_launch_dependents_if_large();
}

template <int R>
static int scan_launch(const DeltaArgs& a, cudaStream_t s) {
  const dim3 grid((a.dv + DELTA_COLS - 1) / DELTA_COLS, a.H, a.n_seqs), block(DELTA_LANES * DELTA_COLS);
  const size_t smem = (size_t)2 * DELTA_TT * (2 * DELTA_LANES * R + DELTA_COLS + 4) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t ce = cudaFuncSetAttribute(delta_scan_kernel<R>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
  }
  return gb_launch(delta_scan_kernel<R>, grid, block, smem, s, a);
}

static int delta_check(const DeltaArgs& a) {
  if (a.n_tokens < 0 || a.n_seqs <= 0 || a.H <= 0 || a.G <= 0 || a.H % a.G || a.dk <= 0 ||
      a.dv <= 0 || a.taps <= 0 || !a.proj || !a.state || !a.prep || !a.o || !a.y)
    return GB_ERR_BAD_ARG;
  if (a.dk > 32 * DELTA_LANES) return GB_ERR_UNSUPPORTED;
  if (a.prep_stride < 2 * a.G * a.dk + a.H * a.dv + 2 * a.H + a.G || (a.prep_stride & 3) ||
      (((uintptr_t)a.prep) & 15))
    return GB_ERR_BAD_ARG;
  return 0;
}

template <typename T>
static int delta_forward(const DeltaArgs& a, cudaStream_t s) {
  int e = delta_check(a);
  if (e) return e;
  if (a.n_tokens == 0) return 0;
  const int Cc = 2 * a.G * a.dk + a.H * a.dv;
  const size_t smem = (size_t)Cc * sizeof(float);
  if (smem > 200 * 1024) return GB_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t ce = cudaFuncSetAttribute(delta_prepare_kernel,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
  }
  e = gb_launch(delta_prepare_kernel, dim3(a.n_tokens), dim3(256), smem, s, a);
  if (e) return e;
  if (a.taps > 1) {
    e = gb_launch(delta_keep_kernel, dim3(a.n_seqs, (Cc + 1023) / 1024), dim3(256), 0, s, a);
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
  return gb_launch(delta_finish_kernel<T>, dim3(a.n_tokens, (a.H + warps - 1) / warps),
                   dim3(warps * 32), 0, s, a);
}

// Four launches: prepare, keep (with more than one tap), scan, finish.
GB_EXPORT int gb_delta_forward_f32(const DeltaArgs* a, cudaStream_t s) { return delta_forward<float>(*a, s); }
GB_EXPORT int gb_delta_forward_bf16(const DeltaArgs* a, cudaStream_t s) { return delta_forward<bf16>(*a, s); }
