// Kernels on a 32-bit residual stream whose norms sit on the sublayers' OUTPUTS:
//   * embedding gather with a scale, written as the fp32 stream and (bf16 path) its rounding,
//   * x' = x + rmsnorm(y) * gamma: the norm of a sublayer's output added to the stream, with the
//     activation-type copy of x' that the next sublayer's products read,
//   * the clamped, sigmoid-gated GLU activation over row-interleaved gate/up values,
// and on one whose norms sit behind the sums:
//   * x' = rmsnorm(alpha * x + y) * gamma, the normed sum being the stream itself; y may be the
//     rows of a routed feed-forward's (token, expert) pairs, added up here in the order chosen.
// Arithmetic is fp32; T is the activation type (float for the 32-bit path, bf16 for serving).
#include "common.cuh"

namespace gf {

// out[t, :] = float(W[ids[t], :]) * scale; act[t, :] = T(out[t, :]) when asked for.
template <typename W, typename T>
__global__ void embedding_scaled_kernel(const int* __restrict__ ids, const W* __restrict__ w,
                                        float scale, float* __restrict__ out, T* __restrict__ act,
                                        int H) {
  const int t = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const W* src = w + (size_t)ids[t] * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = to_f32(src[j]) * scale;
    out[(size_t)t * H + j] = v;
    if (act) act[(size_t)t * H + j] = from_f32<T>(v);
  }
}

// One block per row.  y: the sublayer's output (Y = float or T).  out = x + y * gamma / rms(y) with
// rms = sqrtf(mean(y^2) + eps); act (nullable) = T(out).  out may alias x.
template <typename Y, typename T>
__global__ void outnorm_add_kernel(const float* __restrict__ x, const Y* __restrict__ y,
                                   const float* __restrict__ gamma, float eps,
                                   float* __restrict__ out, T* __restrict__ act, int H) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const size_t base = (size_t)r * H;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = to_f32(y[base + j]);
    row[j] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = x[base + j] + row[j] * gamma[j] / rms;
    out[base + j] = v;
    if (act) act[base + j] = from_f32<T>(v);
  }
}


// The same with four channels an access and the row kept in registers (OPT quads a thread): per row
// this moves what the definition needs and nothing else.  Needs H % 4 == 0 and H <= 4 * OPT * threads.
template <typename Y, typename T, int OPT>
__global__ void outnorm_add_vec_kernel(const float* __restrict__ x, const Y* __restrict__ y,
                                       const float* __restrict__ gamma, float eps,
                                       float* __restrict__ out, T* __restrict__ act, int H) {
  __shared__ float scratch[33];
  const int r = blockIdx.x, nq = H >> 2;
  pdl_trigger();
  float gam[OPT][4], yv[OPT][4];
#pragma unroll
  for (int u = 0; u < OPT; ++u) {                  // weights: before the wait
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) Quad<float>::load(gamma + 4 * q, gam[u]);
  }
  pdl_wait();
  const size_t base = (size_t)r * H;
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < OPT; ++u) {
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) {
      Quad<Y>::load(y + base + 4 * q, yv[u]);
#pragma unroll
      for (int i = 0; i < 4; ++i) ss += yv[u][i] * yv[u][i];
    }
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int u = 0; u < OPT; ++u) {
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) {
      float xv[4];
      Quad<float>::load(x + base + 4 * q, xv);
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] += yv[u][i] * gam[u][i] / rms;
      Quad<float>::store(out + base + 4 * q, xv);
      if (act) Quad<T>::store(act + base + 4 * q, xv);
    }
  }
}

// Norm after the sum.  One block per row: s = alpha * x + y, out = s * gamma / rms(s) with
// rms = sqrtf(mean(s^2) + eps); act (nullable) = T(out).  y: the sublayer's output (Y = float or
// T), or, with pos_of_pair, rows of (token, choice) pairs: y[t] = sum_k wgt[t, k] * rows[pos[t * top
// + k]] (wgt null: 1), added up in the order k = 0, 1, ...  out may alias x.
template <typename Y>
__device__ __forceinline__ float post_y(const Y* __restrict__ y, const int* __restrict__ pos,
                                        const float* __restrict__ wgt, int top, int r, int H,
                                        int j) {
  if (pos == nullptr) return to_f32(y[(size_t)r * H + j]);
  float a = 0.f;
  for (int k = 0; k < top; ++k) {
    const float v = to_f32(y[(size_t)pos[r * top + k] * H + j]);
    a = wgt != nullptr ? fmaf(wgt[r * top + k], v, a) : a + v;
  }
  return a;
}

template <typename Y, typename T>
__global__ void postnorm_kernel(const float* __restrict__ x, const Y* __restrict__ y,
                                const int* __restrict__ pos, const float* __restrict__ wgt,
                                int top, float alpha, const float* __restrict__ gamma, float eps,
                                float* __restrict__ out, T* __restrict__ act, int H) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const size_t base = (size_t)r * H;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = fmaf(alpha, x[base + j], post_y(y, pos, wgt, top, r, H, j));
    row[j] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = row[j] / rms * gamma[j];
    out[base + j] = v;
    if (act) act[base + j] = from_f32<T>(v);
  }
}

// Four channels an access, the row in registers (OPT quads a thread).  H % 4 == 0, H <= 4 * OPT *
// threads, 16-byte aligned rows.
template <typename Y, typename T, int OPT>
__global__ void postnorm_vec_kernel(const float* __restrict__ x, const Y* __restrict__ y,
                                    const int* __restrict__ pos, const float* __restrict__ wgt,
                                    int top, float alpha, const float* __restrict__ gamma,
                                    float eps, float* __restrict__ out, T* __restrict__ act,
                                    int H) {
  __shared__ float scratch[33];
  const int r = blockIdx.x, nq = H >> 2;
  pdl_trigger();
  float gam[OPT][4], sv[OPT][4];
#pragma unroll
  for (int u = 0; u < OPT; ++u) {                  // weights: before the wait
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) Quad<float>::load(gamma + 4 * q, gam[u]);
  }
  pdl_wait();
  const size_t base = (size_t)r * H;
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < OPT; ++u) {
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) {
      float yv[4];
      if (pos == nullptr) {
        Quad<Y>::load(y + base + 4 * q, yv);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) yv[i] = 0.f;
        for (int k = 0; k < top; ++k) {
          float pv[4];
          Quad<Y>::load(y + (size_t)pos[r * top + k] * H + 4 * q, pv);
          const float w = wgt != nullptr ? wgt[r * top + k] : 1.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) yv[i] = wgt != nullptr ? fmaf(w, pv[i], yv[i]) : yv[i] + pv[i];
        }
      }
      Quad<float>::load(x + base + 4 * q, sv[u]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        sv[u][i] = fmaf(alpha, sv[u][i], yv[i]);
        ss += sv[u][i] * sv[u][i];
      }
    }
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int u = 0; u < OPT; ++u) {
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) {
#pragma unroll
      for (int i = 0; i < 4; ++i) sv[u][i] = sv[u][i] / rms * gam[u][i];
      Quad<float>::store(out + base + 4 * q, sv[u]);
      if (act) Quad<T>::store(act + base + 4 * q, sv[u]);
    }
  }
}

// gu[t, 2 i] = gate, gu[t, 2 i + 1] = up.  g = min(gate, limit), u = clamp(up, -limit, limit),
// out = g * sigmoid(alpha * g) * (u + up_shift).
__device__ __forceinline__ float clamped_glu(float g, float u, float limit, float alpha,
                                             float up_shift) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  if (alpha < 0.f) return fmaxf(g, 0.f) * (u + up_shift);   // the sigmoid sharpened to a step: relu
  return g / (1.f + expf(-alpha * g)) * (u + up_shift);
}

template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, size_t total,
                                   float limit, float alpha, float up_shift) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(clamped_glu(to_f32(gu[2 * i]), to_f32(gu[2 * i + 1]), limit, alpha,
                                     up_shift));
}

}  // namespace gf

using namespace gf;
using bf = __nv_bfloat16;

GF_DEFINE_PDL_SWITCH

GF_EXPORT int gf_embedding_scaled(const int* ids, const void* w, int w_dtype, float scale,
                                  float* out, void* act, int act_dtype, int T, int H,
                                  void* stream) {
  if (T <= 0) return 0;
  auto st = (cudaStream_t)stream;
  const dim3 grid(T), block(H >= 1024 ? 256 : 128);
  if (w_dtype == GF_F32) {
    if (act && act_dtype != GF_F32) return -2;
    return launch_kernel(embedding_scaled_kernel<float, float>, grid, block, 0, st, ids,
                         (const float*)w, scale, out, (float*)act, H);
  }
  if (act && act_dtype != GF_BF16) return -2;
  return launch_kernel(embedding_scaled_kernel<bf, bf>, grid, block, 0, st, ids, (const bf*)w,
                       scale, out, (bf*)act, H);
}

GF_EXPORT int gf_outnorm_add(const float* x, const void* y, int y_dtype, const float* gamma,
                             float eps, float* out, void* act, int act_dtype, int R, int H,
                             void* stream) {
  if (R <= 0) return 0;
  auto st = (cudaStream_t)stream;
  const bool al = ((uintptr_t)x | (uintptr_t)y | (uintptr_t)gamma | (uintptr_t)out | (uintptr_t)act) % 16 == 0;
  if (H % 4 == 0 && H <= 4 * 4 * 256 && al) {
    const int nq = H / 4;
    const dim3 vgrid(R), vblock(nq <= 128 ? 128 : 256);
#define GF_VEC(Y, T, OPT)                                                                        \
  return launch_kernel(outnorm_add_vec_kernel<Y, T, OPT>, vgrid, vblock, 0, st, x, (const Y*)y,   \
                       gamma, eps, out, (T*)act, H)
#define GF_OPT(Y, T)                                  \
  {                                                   \
    if (nq <= (int)vblock.x) GF_VEC(Y, T, 1);         \
    if (nq <= 2 * (int)vblock.x) GF_VEC(Y, T, 2);     \
    GF_VEC(Y, T, 4);                                  \
  }
    if (act_dtype == GF_F32) {
      if (y_dtype != GF_F32) return -2;
      GF_OPT(float, float)
    }
    if (y_dtype == GF_F32) GF_OPT(float, bf)
    GF_OPT(bf, bf)
#undef GF_OPT
#undef GF_VEC
  }
  const dim3 grid(R), block(H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 48 * 1024) return -4;
  if (act_dtype == GF_F32) {
    if (y_dtype != GF_F32) return -2;
    return launch_kernel(outnorm_add_kernel<float, float>, grid, block, smem, st, x,
                         (const float*)y, gamma, eps, out, (float*)act, H);
  }
  if (y_dtype == GF_F32)
    return launch_kernel(outnorm_add_kernel<float, bf>, grid, block, smem, st, x, (const float*)y,
                         gamma, eps, out, (bf*)act, H);
  return launch_kernel(outnorm_add_kernel<bf, bf>, grid, block, smem, st, x, (const bf*)y, gamma,
                       eps, out, (bf*)act, H);
}

// x [R, H] fp32; y [R, H] (or, with pos_of_pair [R * top], rows of pairs [P, H]); out may be x.
GF_EXPORT int gf_postnorm(const float* x, const void* y, int y_dtype, const int* pos_of_pair,
                          const float* pair_w, int top, float alpha, const float* gamma, float eps,
                          float* out, void* act, int act_dtype, int R, int H, void* stream) {
  if (R <= 0) return 0;
  auto st = (cudaStream_t)stream;
  const bool al = ((uintptr_t)x | (uintptr_t)y | (uintptr_t)gamma | (uintptr_t)out | (uintptr_t)act) % 16 == 0;
  if (act_dtype == GF_F32 && y_dtype != GF_F32) return -2;
  if (H % 4 == 0 && H <= 4 * 4 * 256 && al) {
    const int nq = H / 4;
    const dim3 vgrid(R), vblock(nq <= 128 ? 128 : 256);
#define GF_VEC(Y, T, OPT)                                                                        \
  return launch_kernel(postnorm_vec_kernel<Y, T, OPT>, vgrid, vblock, 0, st, x, (const Y*)y,      \
                       pos_of_pair, pair_w, top, alpha, gamma, eps, out, (T*)act, H)
#define GF_OPT(Y, T)                                  \
  {                                                   \
    if (nq <= (int)vblock.x) GF_VEC(Y, T, 1);         \
    if (nq <= 2 * (int)vblock.x) GF_VEC(Y, T, 2);     \
    GF_VEC(Y, T, 4);                                  \
  }
    if (act_dtype == GF_F32) GF_OPT(float, float)
    if (y_dtype == GF_F32) GF_OPT(float, bf)
    GF_OPT(bf, bf)
#undef GF_OPT
#undef GF_VEC
  }
  const dim3 grid(R), block(H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 48 * 1024) return -4;
#define GF_GO(Y, T)                                                                              \
  return launch_kernel(postnorm_kernel<Y, T>, grid, block, smem, st, x, (const Y*)y, pos_of_pair, \
                       pair_w, top, alpha, gamma, eps, out, (T*)act, H)
  if (act_dtype == GF_F32) GF_GO(float, float);
  if (y_dtype == GF_F32) GF_GO(float, bf);
  GF_GO(bf, bf);
#undef GF_GO
}

GF_EXPORT int gf_clamped_glu(const void* gu, void* out, int T, int I, float limit, float alpha,
                             float up_shift, int dtype, void* stream) {
  const size_t total = (size_t)T * I;
  if (total == 0) return 0;
  auto st = (cudaStream_t)stream;
  const size_t want = (total + 255) / 256;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == GF_F32)
    return launch_kernel(clamped_glu_kernel<float>, dim3(blocks), dim3(256), 0, st,
                         (const float*)gu, (float*)out, total, limit, alpha, up_shift);
  return launch_kernel(clamped_glu_kernel<bf>, dim3(blocks), dim3(256), 0, st, (const bf*)gu,
                       (bf*)out, total, limit, alpha, up_shift);
}
