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
// the step it is part of.  Norm weights, biases and the offset are 32-bit.
#include "common.cuh"

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

#define LN_VMAX 4   // float4 pieces per thread in the register kernel

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

// Widths that are a multiple of 4 and at most 4 * 1024 * LN_VMAX: a thread keeps
// its values in registers from the first load to the last store.
template <typename T>
__global__ void add_layernorm_vec_kernel(const LayerNormArgs a) {
  __shared__ float scratch[32];
  pdl_launch_dependents_if_small();
  const int N = a.N;
  // weights, biases and the offset are no kernel's output: fetched before the wait
  float wv[LN_VMAX][4], bv[LN_VMAX][4], pw[LN_VMAX][4], pb[LN_VMAX][4], ov[LN_VMAX][4];
#pragma unroll
  for (int j = 0; j < LN_VMAX; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) wv[j][e] = pw[j][e] = 1.f, bv[j][e] = pb[j][e] = ov[j][e] = 0.f;
    if (i < N) {
      if (a.w) LnVec<float>::load(a.w + i, wv[j]);
      if (a.b) LnVec<float>::load(a.b + i, bv[j]);
      if (a.post_w) LnVec<float>::load(a.post_w + i, pw[j]);
      if (a.post_b) LnVec<float>::load(a.post_b + i, pb[j]);
      if (a.offset) LnVec<float>::load(a.offset + i, ov[j]);
    }
  }
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
  if (has_d && a.post_w) {
    float mean = 0.f;
    if (a.post_center) {
      float sm = 0.f;
#pragma unroll
      for (int j = 0; j < LN_VMAX; ++j)
        if ((threadIdx.x + j * blockDim.x) * 4 < N) sm += (dv[j][0] + dv[j][1]) + (dv[j][2] + dv[j][3]);
      mean = block_sum(sm, scratch) * inv_n;
    }
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < LN_VMAX; ++j)
      if ((threadIdx.x + j * blockDim.x) * 4 < N) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          dv[j][e] -= mean;
          sq += dv[j][e] * dv[j][e];
        }
      }
    const float rstd = 1.0f / sqrtf(block_sum(sq, scratch) * inv_n + a.post_eps);
#pragma unroll
    for (int j = 0; j < LN_VMAX; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) dv[j][e] = dv[j][e] * rstd * pw[j][e] + pb[j][e];
  }
  float* rout = a.res_out ? a.res_out + (size_t)r * N : nullptr;
  float sm = 0.f;
#pragma unroll
  for (int j = 0; j < LN_VMAX; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < N) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        av[j][e] = av[j][e] + (has_d ? a.mult * dv[j][e] : 0.f) + ov[j][e];
        sm += av[j][e];
      }
      if (rout) LnVec<float>::store(rout + i, av[j]);
    }
  }
  if (!a.w) {
    pdl_launch_dependents_if_large();
    return;
  }
  const float mean = a.center ? block_sum(sm, scratch) * inv_n : 0.f;
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < LN_VMAX; ++j)
    if ((threadIdx.x + j * blockDim.x) * 4 < N) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        av[j][e] -= mean;
        sq += av[j][e] * av[j][e];
      }
    }
  const float rstd = 1.0f / sqrtf(block_sum(sq, scratch) * inv_n + a.eps);
  pdl_launch_dependents_if_large();
  T* yo = (T*)a.y + (size_t)r * N;
#pragma unroll
  for (int j = 0; j < LN_VMAX; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < N) {
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = av[j][e] * rstd * wv[j][e] + bv[j][e];
      LnVec<T>::store(yo + i, o);
    }
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
  if (a.N % 4 == 0 && a.N <= 4 * 1024 * LN_VMAX && (all & 15) == 0 &&
      ((size_t)a.N * sizeof(T)) % 8 == 0) {
    int threads = (a.N / 4 + LN_VMAX - 1) / LN_VMAX;
    threads = ((threads + 31) / 32) * 32;
    if (threads < 64) threads = 64;
    if (threads > 1024) threads = 1024;
    return gb_launch(add_layernorm_vec_kernel<T>, dim3(a.n_rows), dim3(threads), 0, stream, a);
  }
  int threads = ((a.N + 3) / 4 + 31) / 32 * 32;
  if (threads < 32) threads = 32;
  if (threads > 1024) threads = 1024;
  return gb_launch(add_layernorm_kernel<T>, dim3(a.n_rows), dim3(threads), 0, stream, a);
}

GB_EXPORT int gb_add_layernorm_f32(const LayerNormArgs* a, cudaStream_t s) { return launch<float>(*a, s); }
GB_EXPORT int gb_add_layernorm_bf16(const LayerNormArgs* a, cudaStream_t s) { return launch<bf16>(*a, s); }
