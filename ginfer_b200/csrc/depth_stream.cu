// Kernels of a 32-bit residual stream with norms on both sides of every sublayer and an average
// over the depth of the model:
//   * embedding gather plus a learned row of the token's position, written as the fp32 stream, with
//     the RMS norm of the first sublayer in the same pass,
//   * the end of a sublayer: v = x + y * gamma_b / rms(y) (the norm of the sublayer's output added
//     to the stream); where the layer ends, v is kept as the layer's result and the stream becomes a
//     weighted sum over the embedding output and every layer's result so far,
//     s = sum_j w[j] * X_j (X_n = v, the earlier ones read from the history); then the RMS norm of
//     the next sublayer, n = s * gamma / rms(s), in the activation type.  One block a row.
// Arithmetic is fp32; T is the activation type (float for the 32-bit path, bf16 for serving).
#include "common.cuh"

namespace gf {

template <typename W, typename T>
__global__ void embedding_pos_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                     const W* __restrict__ emb, const W* __restrict__ pos_table,
                                     float* __restrict__ out, const float* __restrict__ gamma,
                                     float eps, T* __restrict__ normed, int H) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const W* e = emb + (size_t)ids[t] * H;
  const W* p = pos_table + (size_t)positions[t] * H;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = to_f32(e[j]) + to_f32(p[j]);
    out[(size_t)t * H + j] = v;
    if (normed) row[j] = v;
    ss += v * v;
  }
  if (!normed) return;
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
  for (int j = threadIdx.x; j < H; j += blockDim.x)
    normed[(size_t)t * H + j] = from_f32<T>(row[j] / rms * gamma[j]);
}

struct DepthMix {
  const float* hist;       // [n, rows, H]: the states before this one (null: no average)
  const float* w;          // [n + 1] weights, the last one for the state just formed
  float* keep;             // where the state just formed goes ([rows, H]; null: nowhere)
  int n;
  size_t stride;           // floats between two states of the history
};

// Generic form: the row in shared memory.
template <typename Y, typename T>
__global__ void sandwich_kernel(const float* __restrict__ x, const Y* __restrict__ y,
                                const float* __restrict__ y_bias,
                                const float* __restrict__ gamma_b, float eps, DepthMix mix,
                                float* __restrict__ out, const float* __restrict__ gamma_next,
                                float eps_next, T* __restrict__ normed, int H) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const size_t base = (size_t)r * H;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = to_f32(y[base + j]) + (y_bias ? y_bias[j] : 0.f);
    row[j] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
  float s2 = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float v = x[base + j] + row[j] * gamma_b[j] / rms;
    if (mix.keep) mix.keep[base + j] = v;
    if (mix.w) {
      float s = 0.f;
      for (int i = 0; i < mix.n; ++i) s = fmaf(mix.w[i], mix.hist[i * mix.stride + base + j], s);
      v = fmaf(mix.w[mix.n], v, s);
    }
    if (out) out[base + j] = v;
    row[j] = v;
    s2 += v * v;
  }
  if (!normed) return;
  s2 = block_sum(s2, scratch);
  const float rms2 = sqrtf(s2 / (float)H + eps_next);
  for (int j = threadIdx.x; j < H; j += blockDim.x)
    normed[base + j] = from_f32<T>(row[j] / rms2 * gamma_next[j]);
}

// Four channels an access, the row in registers (OPT quads a thread): H % 4 == 0, H <= 4 * OPT *
// threads, 16-byte aligned rows.
template <typename Y, typename T, int OPT>
__global__ void sandwich_vec_kernel(const float* __restrict__ x, const Y* __restrict__ y,
                                    const float* __restrict__ y_bias,
                                    const float* __restrict__ gamma_b, float eps, DepthMix mix,
                                    float* __restrict__ out, const float* __restrict__ gamma_next,
                                    float eps_next, T* __restrict__ normed, int H) {
  __shared__ float scratch[33];
  const int r = blockIdx.x, nq = H >> 2;
  pdl_trigger();
  float gam[OPT][4], v[OPT][4];
#pragma unroll
  for (int u = 0; u < OPT; ++u) {                  // weights: before the wait
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) Quad<float>::load(gamma_b + 4 * q, gam[u]);
  }
  pdl_wait();
  const size_t base = (size_t)r * H;
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < OPT; ++u) {
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) {
      Quad<Y>::load(y + base + 4 * q, v[u]);
      if (y_bias) {
        float b[4];
        Quad<float>::load(y_bias + 4 * q, b);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[u][i] += b[i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) ss += v[u][i] * v[u][i];
    }
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
  float s2 = 0.f;
#pragma unroll
  for (int u = 0; u < OPT; ++u) {
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) {
      float xv[4];
      Quad<float>::load(x + base + 4 * q, xv);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[u][i] = xv[i] + v[u][i] * gam[u][i] / rms;
      if (mix.keep) Quad<float>::store(mix.keep + base + 4 * q, v[u]);
      if (mix.w) {
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < mix.n; ++k) {
          float hv[4];
          Quad<float>::load(mix.hist + k * mix.stride + base + 4 * q, hv);
          const float wk = mix.w[k];
#pragma unroll
          for (int i = 0; i < 4; ++i) s[i] = fmaf(wk, hv[i], s[i]);
        }
        const float wn = mix.w[mix.n];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[u][i] = fmaf(wn, v[u][i], s[i]);
      }
      if (out) Quad<float>::store(out + base + 4 * q, v[u]);
#pragma unroll
      for (int i = 0; i < 4; ++i) s2 += v[u][i] * v[u][i];
    }
  }
  if (!normed) return;
#pragma unroll
  for (int u = 0; u < OPT; ++u) {                  // the next norm's weights
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) Quad<float>::load(gamma_next + 4 * q, gam[u]);
  }
  s2 = block_sum(s2, scratch);
  const float rms2 = sqrtf(s2 / (float)H + eps_next);
#pragma unroll
  for (int u = 0; u < OPT; ++u) {
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) {
#pragma unroll
      for (int i = 0; i < 4; ++i) v[u][i] = v[u][i] / rms2 * gam[u][i];
      Quad<T>::store(normed + base + 4 * q, v[u]);
    }
  }
}

}  // namespace gf

using namespace gf;
using bf = __nv_bfloat16;

GF_DEFINE_PDL_SWITCH

// ids, positions: [T]; emb [vocab, H], pos_table [positions, H] of one type (w_dtype); out [T, H]
// fp32; gamma / normed: the first norm's weight (fp32) and its result in act_dtype, or null.
GF_EXPORT int gf_embedding_pos(const int* ids, const int* positions, const void* emb,
                               const void* pos_table, int w_dtype, float* out, const float* gamma,
                               float eps, void* normed, int act_dtype, int T, int H, void* stream) {
  if (T <= 0) return 0;
  auto st = (cudaStream_t)stream;
  const dim3 grid(T), block(H >= 1024 ? 256 : 128);
  const size_t smem = normed ? (size_t)H * sizeof(float) : 0;
  if (smem > 48 * 1024) return -4;
  if (w_dtype == GF_F32) {
    if (normed && act_dtype != GF_F32) return -2;
    return launch_kernel(embedding_pos_kernel<float, float>, grid, block, smem, st, ids, positions,
                         (const float*)emb, (const float*)pos_table, out, gamma, eps,
                         (float*)normed, H);
  }
  if (normed && act_dtype != GF_BF16) return -2;
  return launch_kernel(embedding_pos_kernel<bf, bf>, grid, block, smem, st, ids, positions,
                       (const bf*)emb, (const bf*)pos_table, out, gamma, eps, (bf*)normed, H);
}

// x [R, H] fp32, y [R, H] in y_dtype (y_bias, nullable fp32 [H], is added to every row of y first: the
// bias of a product whose library kernel has no epilogue for it), gamma_b fp32.  hist / mix_w / n_hist / hist_stride / keep: the
// depth average (mix_w null: none).  out (nullable) [R, H] fp32: the stream afterwards.
// gamma_next / normed (nullable): the next norm in act_dtype.
GF_EXPORT int gf_sandwich_update(const float* x, const void* y, int y_dtype, const float* y_bias,
                                 const float* gamma_b,
                                 float eps, const float* hist, const float* mix_w, int n_hist,
                                 long long hist_stride, float* keep, float* out,
                                 const float* gamma_next, float eps_next, void* normed, int act_dtype,
                                 int R,
                                 int H, void* stream) {
  if (R <= 0) return 0;
  if (act_dtype == GF_F32 && y_dtype != GF_F32) return -2;
  auto st = (cudaStream_t)stream;
  DepthMix mix{hist, mix_w, keep, mix_w ? n_hist : 0, (size_t)hist_stride};
  const bool al = ((uintptr_t)x | (uintptr_t)y | (uintptr_t)y_bias | (uintptr_t)gamma_b | (uintptr_t)out |
                   (uintptr_t)keep | (uintptr_t)hist | (uintptr_t)gamma_next |
                   (uintptr_t)normed) % 16 == 0 && hist_stride % 4 == 0;
  if (H % 4 == 0 && H <= 4 * 4 * 256 && al) {
    const int nq = H / 4;
    const dim3 vgrid(R), vblock(nq <= 128 ? 128 : 256);
#define GF_VEC(Y, T, OPT)                                                                        \
  return launch_kernel(sandwich_vec_kernel<Y, T, OPT>, vgrid, vblock, 0, st, x, (const Y*)y,      \
                       y_bias, gamma_b, eps, mix, out, gamma_next, eps_next, (T*)normed, H)
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
  return launch_kernel(sandwich_kernel<Y, T>, grid, block, smem, st, x, (const Y*)y, y_bias,      \
                       gamma_b, eps, mix, out, gamma_next, eps_next, (T*)normed, H)
  if (act_dtype == GF_F32) GF_GO(float, float);
  if (y_dtype == GF_F32) GF_GO(float, bf);
  GF_GO(bf, bf);
#undef GF_GO
}
