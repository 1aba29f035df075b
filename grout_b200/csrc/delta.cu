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
//            16 columns a block, and a sequence's rows are walked in order; the
//            next token's operands are fetched while the current one is worked.
//            A token's result does not depend on how the sequence was cut into
//            steps: the order of operations is the same.
//   finish   one warp per (token, head): norm over dv, weight, gate
//
// Columns of the projection: q [G dk] | k [G dk] | v [H dv] | gate [H dv] | b [H] | a [H].
// A sequence's state is one row of floats: the tail [taps - 1, Cc] (Cc = the
// convolved channels q | k | v), then S as [H, dv, dk], a column's dk elements
// side by side.  Rows of slot < 0 (padding) read zeros and store nothing.
#include "common.cuh"

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
  float* prep;             // [n_tokens, Cc + 2 H]: unit q | unit k | v | beta | decay
  float* o;                // [n_tokens, H, dv]
  void* y;                 // [n_tokens, H dv] in the activation type
  int n_tokens, n_seqs, H, G, dk, dv, taps;
  float unit_eps, norm_eps;
};

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__global__ void delta_prepare_kernel(const DeltaArgs a) {
  extern __shared__ float row[];   // [Cc]
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int H = a.H, G = a.G, dk = a.dk, dv = a.dv, taps = a.taps;
  const int Cc = 2 * G * dk + H * dv, C_all = Cc + H * dv + 2 * H, P = Cc + 2 * H;
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
  for (int head = warp; head < 2 * G; head += nwarps) {
    const float* x = row + head * dk;
    float ss = 0.f;
    for (int d = lane; d < dk; d += 32) ss += x[d] * x[d];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss + a.unit_eps);
    const float mul = head < G ? rsqrtf((float)dk) : 1.0f;
    for (int d = lane; d < dk; d += 32) out[head * dk + d] = head < G ? x[d] * inv * mul : x[d] * inv;
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

template <int R>
__global__ void __launch_bounds__(DELTA_LANES * DELTA_COLS) delta_scan_kernel(const DeltaArgs a) {
  pdl_launch_dependents_if_small();
  const int seq = blockIdx.z, h = blockIdx.y;
  const int col = blockIdx.x * DELTA_COLS + threadIdx.x / DELTA_LANES, l = threadIdx.x % DELTA_LANES;
  const int H = a.H, G = a.G, dk = a.dk, dv = a.dv;
  const int Cc = 2 * G * dk + H * dv, P = Cc + 2 * H;
  const int kvh = h / (H / G);
  const bool active = col < dv;
  pdl_wait();
  const int row0 = a.cu_q[seq], n = a.cu_q[seq + 1] - row0;
  if (n <= 0) return;
  const int slot = a.slots[seq];
  float* sp = slot >= 0 && active
                  ? a.state + (size_t)slot * a.state_stride + (size_t)(a.taps - 1) * Cc +
                        ((size_t)h * dv + col) * dk
                  : nullptr;
  float S[R], k[R], q[R], kn[R], qn[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int e = i * DELTA_LANES + l;
    S[i] = sp && e < dk ? sp[e] : 0.f;
  }
  float v, beta, g, vn = 0.f, bn = 0.f, gn = 0.f;
  auto fetch = [&](int t, float (&kk)[R], float (&qq)[R], float& vv, float& bb, float& gg) {
    const float* base = a.prep + (size_t)t * P;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int e = i * DELTA_LANES + l;
      qq[i] = e < dk ? base[kvh * dk + e] : 0.f;
      kk[i] = e < dk ? base[(G + kvh) * dk + e] : 0.f;
    }
    vv = active ? base[2 * G * dk + h * dv + col] : 0.f;
    bb = base[Cc + h];
    gg = base[Cc + H + h];
  };
  fetch(row0, kn, qn, vn, bn, gn);
  for (int t = row0; t < row0 + n; ++t) {
#pragma unroll
    for (int i = 0; i < R; ++i) k[i] = kn[i], q[i] = qn[i];
    v = vn, beta = bn, g = gn;
    if (t + 1 < row0 + n) fetch(t + 1, kn, qn, vn, bn, gn);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) dot = fmaf(S[i], k[i], dot);
#pragma unroll
    for (int m = 1; m < DELTA_LANES; m <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, m);
    const float u = beta * (v - g * dot);
    float rd = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      S[i] = fmaf(k[i], u, g * S[i]);
      rd = fmaf(S[i], q[i], rd);
    }
#pragma unroll
    for (int m = 1; m < DELTA_LANES; m <<= 1) rd += __shfl_xor_sync(0xffffffffu, rd, m);
    if (l == 0 && active) a.o[((size_t)t * H + h) * dv + col] = rd;
  }
  pdl_launch_dependents_if_large();
  if (sp) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int e = i * DELTA_LANES + l;
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

static int delta_check(const DeltaArgs& a) {
  if (a.n_tokens < 0 || a.n_seqs <= 0 || a.H <= 0 || a.G <= 0 || a.H % a.G || a.dk <= 0 ||
      a.dv <= 0 || a.taps <= 0 || !a.proj || !a.state || !a.prep || !a.o || !a.y)
    return GB_ERR_BAD_ARG;
  if (a.dk > 32 * DELTA_LANES) return GB_ERR_UNSUPPORTED;
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
  const dim3 grid((a.dv + DELTA_COLS - 1) / DELTA_COLS, a.H, a.n_seqs), block(DELTA_LANES * DELTA_COLS);
  const int per_lane = (a.dk + DELTA_LANES - 1) / DELTA_LANES;
  if (per_lane <= 4) e = gb_launch(delta_scan_kernel<4>, grid, block, 0, s, a);
  else if (per_lane <= 8) e = gb_launch(delta_scan_kernel<8>, grid, block, 0, s, a);
  else if (per_lane <= 12) e = gb_launch(delta_scan_kernel<12>, grid, block, 0, s, a);
  else if (per_lane <= 16) e = gb_launch(delta_scan_kernel<16>, grid, block, 0, s, a);
  else if (per_lane <= 24) e = gb_launch(delta_scan_kernel<24>, grid, block, 0, s, a);
  else e = gb_launch(delta_scan_kernel<32>, grid, block, 0, s, a);
  if (e) return e;
  const int warps = a.H < 8 ? a.H : 8;
  return gb_launch(delta_finish_kernel<T>, dim3(a.n_tokens, (a.H + warps - 1) / warps),
                   dim3(warps * 32), 0, s, a);
}

// Four launches: prepare, keep (with more than one tap), scan, finish.
GB_EXPORT int gb_delta_forward_f32(const DeltaArgs* a, cudaStream_t s) { return delta_forward<float>(*a, s); }
GB_EXPORT int gb_delta_forward_bf16(const DeltaArgs* a, cudaStream_t s) { return delta_forward<bf16>(*a, s); }
