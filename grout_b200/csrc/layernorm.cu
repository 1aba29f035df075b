// Layer norm with everything a "sandwich" layer does around it folded in.
//
//   d   = delta[s, :]  (or the sum of n_parts 32-bit partial sums of it)
//   c   = post ? mult * (norm(d; post_w, post_b, post_eps)) : mult * d
//   v   = res_in[s, :] + c + offset          (each term may be absent; 32-bit sums)
//   res_out[r, :] = v                        (32-bit residual stream, optional)
//   y[r, :] = norm(v; w, b, eps)             (optional: without w the kernel only adds)
//
//   norm(x; w, b, eps) = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b
//
// with the mean left at zero for a norm that does not centre, and b absent for a
// norm without bias.  s = rows[r] when a row list is given (the gather before
// the final norm), else r.  Means and variances are taken in two passes over
// values that stay in registers (or are recomputed), all in 32-bit; the block's
// tree of sums depends on the width only, so a row's result does not depend on
// the step it is part of (the kernels for bfloat16 activations take a row's sum
// and sum of squares together instead, see below).  Norm weights, biases and the
// offset are 32-bit.
#include <cooperative_groups.h>

#include <type_traits>

#include "common.cuh"

namespace cg = cooperative_groups;

struct LayerNormArgs {
  const float* res_in;
  const void* delta;        // [rows_total, N] in the activation type, or null
  const float* parts;       // instead of delta: n_parts partial sums, part_stride floats apart
  int n_parts;
  long long part_stride;
  const int* rows;          // row list or null
  const float* post_w;      // the norm behind the sublayer that made delta, or null
  const float* post_b;
  float post_eps;
  int post_center;
  float mult;
  const float* offset;      // [N] or null
  const float* w;           // the norm in front of the next sublayer, or null
  const float* b;
  float eps;
  int center;
  float* res_out;
  void* y;
  int n_rows, N;
};

#define LN_VMAX_MOST 4   // float4 pieces per thread in the register kernel, at most

template <typename T> struct LnVec;
template <> struct LnVec<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct LnVec<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float (&v)[4]) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  }
  static __device__ __forceinline__ void store(bf16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 x;
    x.x = *reinterpret_cast<uint32_t*>(&a);
    x.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = x;
  }
};

// Block-wide sums of two values at once with a fixed tree (one pair of barriers).
__device__ __forceinline__ float2 block_sum2(float x, float y, float2* scratch2) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  x = warp_sum(x), y = warp_sum(y);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch2[warp] = make_float2(x, y);
  __syncthreads();
  float2 r = (lane < nwarps) ? scratch2[lane] : make_float2(0.f, 0.f);
  r.x = warp_sum(r.x), r.y = warp_sum(r.y);
  return r;
}

// Widths that are a multiple of 4 and at most 16,384: a thread keeps its values
// (LN_VMAX pieces of four) in registers from the first load to the last store.
// The kernel is a chain of dependent steps (loads, the sums over the row, stores),
// so what it reaches is set by how many rows an SM has in flight: blocks are kept
// small (a row of 2,560 is 160 threads with four pieces each) and norm weights are
// read where they are used, not held from the start, which keeps the registers
// at 64 a thread and six or more rows on an SM.  (One piece a thread, 640 threads
// and weights held in registers left one row on an SM: 2.6 times the time.)
// In 32-bit the mean is taken first and the deviations are squared (two sums per
// norm); with bfloat16 activations sum and sum of squares are taken together (one
// sum per norm, var = E[x^2] - mean^2 in 32-bit), which halves the chain.
template <typename T, int LN_VMAX>
__global__ void __launch_bounds__(1024) add_layernorm_vec_kernel(const LayerNormArgs a) {
  __shared__ float2 scratch2[32];
  float* scratch = reinterpret_cast<float*>(scratch2);
  constexpr bool TWO_PASS = std::is_same<T, float>::value;
  pdl_launch_dependents_if_small();
  const int N = a.N;
  pdl_wait();
  const int r = blockIdx.x;
  const size_t s = a.rows ? (size_t)a.rows[r] : (size_t)r;
  const float* rin = a.res_in ? a.res_in + s * N : nullptr;
  const T* din = a.delta ? (const T*)a.delta + s * N : nullptr;
  const float* pin = a.parts ? a.parts + s * N : nullptr;
  const bool has_d = din || pin;
  float av[LN_VMAX][4], dv[LN_VMAX][4];
#pragma unroll
  for (int j = 0; j < LN_VMAX; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) av[j][e] = dv[j][e] = 0.f;
    if (i < N) {
      if (rin) LnVec<float>::load(rin + i, av[j]);
      if (din) LnVec<T>::load(din + i, dv[j]);
    }
  }
  if (pin) {
#pragma unroll
    for (int j = 0; j < LN_VMAX; ++j) {
      const int i = (threadIdx.x + j * blockDim.x) * 4;
      if (i < N) {
        for (int k0 = 0; k0 < a.n_parts; k0 += 4) {   // four requested at once, added in order
          float pk[4][4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int k = k0 + u < a.n_parts ? k0 + u : a.n_parts - 1;
            LnVec<float>::load(pin + (size_t)k * a.part_stride + i, pk[u]);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (k0 + u < a.n_parts) {
#pragma unroll
              for (int e = 0; e < 4; ++e) dv[j][e] += pk[u][e];
            }
        }
      }
    }
  }
  const float inv_n = 1.0f / (float)N;
  // mean and 1 / sqrt(var + eps) of the row whose pieces are x
  auto row_stats = [&](const float (&x)[LN_VMAX][4], bool center, float eps, float& mean, float& rstd) {
    float sm = 0.f, sq = 0.f;
#pragma unroll
    for (int j = 0; j < LN_VMAX; ++j)
      if ((threadIdx.x + j * blockDim.x) * 4 < N) {
        sm += (x[j][0] + x[j][1]) + (x[j][2] + x[j][3]);
        if (!TWO_PASS) sq += (x[j][0] * x[j][0] + x[j][1] * x[j][1]) + (x[j][2] * x[j][2] + x[j][3] * x[j][3]);
      }
    if (TWO_PASS) {
      mean = center ? block_sum(sm, scratch) * inv_n : 0.f;
#pragma unroll
      for (int j = 0; j < LN_VMAX; ++j)
        if ((threadIdx.x + j * blockDim.x) * 4 < N) {
#pragma unroll
          for (int e = 0; e < 4; ++e) sq += (x[j][e] - mean) * (x[j][e] - mean);
        }
      rstd = 1.0f / sqrtf(block_sum(sq, scratch) * inv_n + eps);
    } else {
      const float2 t = block_sum2(sm, sq, scratch2);
      mean = center ? t.x * inv_n : 0.f;
      rstd = 1.0f / sqrtf(fmaxf(t.y * inv_n - mean * mean, 0.f) + eps);
    }
  };
  if (has_d && a.post_w) {
    float mean, rstd;
    row_stats(dv, a.post_center != 0, a.post_eps, mean, rstd);
#pragma unroll
    for (int j = 0; j < LN_VMAX; ++j) {
      const int i = (threadIdx.x + j * blockDim.x) * 4;
      if (i < N) {
        float pw[4], pb[4] = {0.f, 0.f, 0.f, 0.f};
        LnVec<float>::load(a.post_w + i, pw);
        if (a.post_b) LnVec<float>::load(a.post_b + i, pb);
#pragma unroll
        for (int e = 0; e < 4; ++e) dv[j][e] = (dv[j][e] - mean) * rstd * pw[e] + pb[e];
      }
    }
  }
  float* rout = a.res_out ? a.res_out + (size_t)r * N : nullptr;
#pragma unroll
  for (int j = 0; j < LN_VMAX; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < N) {
      float ov[4] = {0.f, 0.f, 0.f, 0.f};
      if (a.offset) LnVec<float>::load(a.offset + i, ov);
#pragma unroll
      for (int e = 0; e < 4; ++e) av[j][e] = av[j][e] + (has_d ? a.mult * dv[j][e] : 0.f) + ov[e];
      if (rout) LnVec<float>::store(rout + i, av[j]);
    }
  }
  if (!a.w) {
    pdl_launch_dependents_if_large();
    return;
  }
  float mean, rstd;
  row_stats(av, a.center != 0, a.eps, mean, rstd);
  pdl_launch_dependents_if_large();
  T* yo = (T*)a.y + (size_t)r * N;
#pragma unroll
  for (int j = 0; j < LN_VMAX; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < N) {
      float wv[4], bv[4] = {0.f, 0.f, 0.f, 0.f}, o[4];
      LnVec<float>::load(a.w + i, wv);
      if (a.b) LnVec<float>::load(a.b + i, bv);
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = (av[j][e] - mean) * rstd * wv[e] + bv[e];
      LnVec<T>::store(yo + i, o);
    }
  }
}

// A handful of rows (a decode step) would keep a handful of SMs busy, each with a
// long chain of dependent loads.  Here a cluster of LN_CLUSTER blocks shares a
// row: each block owns a quarter of the columns, takes the mean and the sum of
// squared deviations of its quarter, and the quarters' pairs meet through
// distributed shared memory, where they are combined exactly (the mean of the
// means; the sums of squares plus each quarter's n (mean_q - mean)^2), in rank
// order.  One cluster barrier per norm; no block spins on memory.
#define LN_CLUSTER 4
template <typename T>
__global__ void add_layernorm_cluster_kernel(const LayerNormArgs a) {
  __shared__ float scratch[32];
  __shared__ float stat[2][LN_CLUSTER][2];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  pdl_launch_dependents_if_small();
  const int N = a.N, cols = N / LN_CLUSTER;       // a multiple of 4
  const int i = rank * cols + threadIdx.x * 4;    // this thread's four columns
  const bool active = threadIdx.x * 4 < cols;
  float wv[4] = {1.f, 1.f, 1.f, 1.f}, bv[4] = {0.f, 0.f, 0.f, 0.f}, pw[4] = {1.f, 1.f, 1.f, 1.f},
        pb[4] = {0.f, 0.f, 0.f, 0.f}, ov[4] = {0.f, 0.f, 0.f, 0.f};
  if (active) {   // no kernel's output: before the wait
    if (a.w) LnVec<float>::load(a.w + i, wv);
    if (a.b) LnVec<float>::load(a.b + i, bv);
    if (a.post_w) LnVec<float>::load(a.post_w + i, pw);
    if (a.post_b) LnVec<float>::load(a.post_b + i, pb);
    if (a.offset) LnVec<float>::load(a.offset + i, ov);
  }
  pdl_wait();
  const int r = blockIdx.x / LN_CLUSTER;
  const size_t s = a.rows ? (size_t)a.rows[r] : (size_t)r;
  const bool has_d = a.delta || a.parts;
  float av[4] = {0.f, 0.f, 0.f, 0.f}, dv[4] = {0.f, 0.f, 0.f, 0.f};
  if (active) {
    if (a.res_in) LnVec<float>::load(a.res_in + s * N + i, av);
    if (a.delta) LnVec<T>::load((const T*)a.delta + s * N + i, dv);
    // eight partials are requested at once and then added in order (a product is split at
    // most eight ways, so this is one trip to L2)
    for (int k0 = 0; k0 < a.n_parts; k0 += 8) {
      float pk[8][4];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int k = k0 + u < a.n_parts ? k0 + u : a.n_parts - 1;
        LnVec<float>::load(a.parts + (size_t)k * a.part_stride + s * N + i, pk[u]);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (k0 + u < a.n_parts) {
#pragma unroll
          for (int e = 0; e < 4; ++e) dv[e] += pk[u][e];
        }
    }
  }
  // mean and 1 / sqrt(var + eps) of the whole row from this block's quarter x[0..3]
  auto row_stats = [&](int round, const float (&x)[4], bool center, float eps, float& mean, float& rstd) {
    float mean_q = 0.f;
    if (center) mean_q = block_sum(active ? (x[0] + x[1]) + (x[2] + x[3]) : 0.f, scratch) / (float)cols;
    float sq = 0.f;
    if (active) {
#pragma unroll
      for (int e = 0; e < 4; ++e) sq += (x[e] - mean_q) * (x[e] - mean_q);
    }
    const float m2_q = block_sum(sq, scratch);
    // every block puts its pair into every block's table (thread k writes to block k): after
    // the one barrier each block reads its own shared memory only
    if (threadIdx.x < LN_CLUSTER) {
      float* dst = cluster.map_shared_rank(&stat[round][0][0], threadIdx.x);
      dst[rank * 2] = mean_q;
      dst[rank * 2 + 1] = m2_q;
    }
    cluster.sync();
    float msum = 0.f;
#pragma unroll
    for (int k = 0; k < LN_CLUSTER; ++k) msum += stat[round][k][0];
    mean = msum / (float)LN_CLUSTER;
    float m2 = 0.f;
#pragma unroll
    for (int k = 0; k < LN_CLUSTER; ++k) {
      const float dm = stat[round][k][0] - mean;
      m2 += stat[round][k][1] + (float)cols * dm * dm;
    }
    rstd = 1.0f / sqrtf(m2 / (float)N + eps);
  };
  if (has_d && a.post_w) {   // (the same for every block of the cluster)
    float mean, rstd;
    row_stats(0, dv, a.post_center != 0, a.post_eps, mean, rstd);
#pragma unroll
    for (int e = 0; e < 4; ++e) dv[e] = (dv[e] - mean) * rstd * pw[e] + pb[e];
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) av[e] = av[e] + (has_d ? a.mult * dv[e] : 0.f) + ov[e];
  if (active && a.res_out) LnVec<float>::store(a.res_out + (size_t)r * N + i, av);
  if (!a.w) return;
  float mean, rstd;
  row_stats(1, av, a.center != 0, a.eps, mean, rstd);
  if (active) {
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = (av[e] - mean) * rstd * wv[e] + bv[e];
    LnVec<T>::store((T*)a.y + (size_t)r * N + i, o);
  }
}

// Any width: values are recomputed from memory in every pass (the row is in L1).
template <typename T>
__global__ void add_layernorm_kernel(const LayerNormArgs a) {
  __shared__ float scratch[32];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int N = a.N;
  const int r = blockIdx.x;
  const size_t s = a.rows ? (size_t)a.rows[r] : (size_t)r;
  const float* rin = a.res_in ? a.res_in + s * N : nullptr;
  const T* din = a.delta ? (const T*)a.delta + s * N : nullptr;
  const float* pin = a.parts ? a.parts + s * N : nullptr;
  const bool has_d = din || pin;
  const float inv_n = 1.0f / (float)N;
  auto dval = [&](int i) {
    float d = din ? to_f32<T>(din[i]) : 0.f;
    for (int k = 0; k < a.n_parts; ++k) d += pin[(size_t)k * a.part_stride + i];
    return d;
  };
  float pmean = 0.f, prstd = 1.f;
  if (has_d && a.post_w) {
    if (a.post_center) {
      float sm = 0.f;
      for (int i = threadIdx.x; i < N; i += blockDim.x) sm += dval(i);
      pmean = block_sum(sm, scratch) * inv_n;
    }
    float sq = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
      const float d = dval(i) - pmean;
      sq += d * d;
    }
    prstd = 1.0f / sqrtf(block_sum(sq, scratch) * inv_n + a.post_eps);
  }
  auto value = [&](int i) {
    float c = 0.f;
    if (has_d) {
      c = dval(i);
      if (a.post_w) c = (c - pmean) * prstd * a.post_w[i] + (a.post_b ? a.post_b[i] : 0.f);
      c *= a.mult;
    }
    return (rin ? rin[i] : 0.f) + c + (a.offset ? a.offset[i] : 0.f);
  };
  // The stream may be updated in place, so every value is computed once, kept in
  // res_out when there is one, and read back by the thread that stored it.
  float* rout = a.res_out ? a.res_out + (size_t)r * N : nullptr;
  float sm = 0.f;
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    const float v = value(i);
    if (rout) rout[i] = v;
    sm += v;
  }
  if (!a.w) {
    pdl_launch_dependents_if_large();
    return;
  }
  const bool reread = rout != nullptr;
  const float mean = a.center ? block_sum(sm, scratch) * inv_n : 0.f;
  float sq = 0.f;
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    const float v = (reread ? rout[i] : value(i)) - mean;
    sq += v * v;
  }
  const float rstd = 1.0f / sqrtf(block_sum(sq, scratch) * inv_n + a.eps);
  pdl_launch_dependents_if_large();
  T* yo = (T*)a.y + (size_t)r * N;
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    const float v = (reread ? rout[i] : value(i)) - mean;
    yo[i] = from_f32<T>(v * rstd * a.w[i] + (a.b ? a.b[i] : 0.f));
  }
}

template <typename T>
static int launch(const LayerNormArgs& a, cudaStream_t stream) {
  if (a.n_rows < 0 || a.N <= 0 || (!a.res_in && !a.delta && !a.parts && !a.offset)) return GB_ERR_BAD_ARG;
  if ((a.parts != nullptr) != (a.n_parts > 0) || a.n_parts < 0 || (a.parts && a.delta)) return GB_ERR_BAD_ARG;
  if ((a.w != nullptr) != (a.y != nullptr)) return GB_ERR_BAD_ARG;
  if (!a.w && !a.res_out) return GB_ERR_BAD_ARG;
  if (a.post_b && !a.post_w) return GB_ERR_BAD_ARG;
  // in place is allowed only without a row list (each block then owns its row)
  if (a.rows && a.res_out && a.res_out == a.res_in) return GB_ERR_BAD_ARG;
  if (a.n_rows == 0) return 0;
  const uintptr_t all = (uintptr_t)a.res_in | (uintptr_t)a.delta | (uintptr_t)a.parts |
                        (uintptr_t)a.post_w | (uintptr_t)a.post_b | (uintptr_t)a.offset |
                        (uintptr_t)a.w | (uintptr_t)a.b | (uintptr_t)a.res_out | (uintptr_t)a.y |
                        (uintptr_t)(a.part_stride * 4);
  const bool vec_ok = a.N % 4 == 0 && (all & 15) == 0 && ((size_t)a.N * sizeof(T)) % 8 == 0;
  // The cluster kernel is chosen by the number of rows and sums in another order than
  // the kernels below.  The 32-bit path never takes it: there the order of a row's sums
  // may depend on the width alone, so that a token's result is the same in a step of one
  // row and in a step of thousands.
  constexpr bool by_rows_too = !std::is_same<T, float>::value;
  if (by_rows_too && vec_ok && a.n_rows <= 64 && a.N >= 1024 && a.N % (4 * LN_CLUSTER) == 0 &&
      a.N / LN_CLUSTER <= 4096) {
    const int threads = ((a.N / LN_CLUSTER / 4 + 31) / 32) * 32;
    return gb_launch_cluster(add_layernorm_cluster_kernel<T>, dim3(a.n_rows * LN_CLUSTER), dim3(threads),
                             0, stream, LN_CLUSTER, a);
  }
  if (vec_ok && a.N <= 4 * 1024 * LN_VMAX_MOST) {
    const int vmax = a.N <= 1024 ? 1 : (a.N <= 2048 ? 2 : 4);
    int threads = (a.N / 4 + vmax - 1) / vmax;
    threads = ((threads + 31) / 32) * 32;
    if (threads < 64) threads = 64;
    if (threads > 1024) threads = 1024;
    switch (vmax) {
      case 1: return gb_launch(add_layernorm_vec_kernel<T, 1>, dim3(a.n_rows), dim3(threads), 0, stream, a);
      case 2: return gb_launch(add_layernorm_vec_kernel<T, 2>, dim3(a.n_rows), dim3(threads), 0, stream, a);
      default: return gb_launch(add_layernorm_vec_kernel<T, 4>, dim3(a.n_rows), dim3(threads), 0, stream, a);
    }
  }
  int threads = ((a.N + 3) / 4 + 31) / 32 * 32;
  if (threads < 32) threads = 32;
  if (threads > 1024) threads = 1024;
  return gb_launch(add_layernorm_kernel<T>, dim3(a.n_rows), dim3(threads), 0, stream, a);
}

GB_EXPORT int gb_add_layernorm_f32(const LayerNormArgs* a, cudaStream_t s) { return launch<float>(*a, s); }
GB_EXPORT int gb_add_layernorm_bf16(const LayerNormArgs* a, cudaStream_t s) { return launch<bf16>(*a, s); }
