// Kernels of layers that normalise their sublayers' INPUTS on a 32-bit residual stream and scale
// what the sublayers return:
//   * stream_update_kernel   x' = x (+ a second stream) (+ a row vector) + m * f(y), where y is a
//                            sublayer's output and f(y) is y times a per-channel scale or
//                            y / rms(y) times a weight; x' leaves as the fp32 stream, as its
//                            rounding to the activation type, and as norm(x') for the sublayer
//                            that follows (layer norm with weight and bias, or RMS norm), each
//                            only where asked for.  Row selection for the final norm.  y may
//                            also be the rows of a routed feed-forward's (token, expert) pairs:
//                            the kernel then adds up a token's pairs itself, in the order chosen.
//   * qk_norm_rope_kernel    per (token, head): RMS norm over the head's channels with one weight
//                            vector for all heads, rotation of channel pairs by position * f_i
//                            (neighbouring pairs (2i, 2i+1) or halves (i, i + n)), q in place,
//                            k into its cache slot; the values (the keys as projected, or the
//                            columns of a value projection) into theirs.
//   * head_gate_kernel       o[t, h, :] *= sigmoid(g[t, h]).
//   * token_gate_kernel      g[t, j] = gelu_tanh(z[t, j]) * E[token[t], off + j].
// Arithmetic is fp32; T is the activation type (float for the 32-bit path, bf16 for serving).
#include "common.cuh"

namespace gf {

// One block per output row r (source row rows[r] or r).  Shared memory: H floats.
//   ymode 0: no y.  1: + m * scale[j] * y[j] (scale nullable = 1).  2: + m * y[j] / rms(y) * scale[j].
//   norm  0: none.  1: (x' - mean) / sqrt(var + eps) * w + b (b nullable).  2: x' / rms(x') * w.
template <typename Y, typename T>
__global__ void stream_update_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                     const Y* __restrict__ y, int ymode,
                                     const float* __restrict__ scale, float m, float y_eps,
                                     const float* __restrict__ add_full,
                                     const float* __restrict__ add_row, float* __restrict__ out,
                                     T* __restrict__ act, int norm, const float* __restrict__ nw,
                                     const float* __restrict__ nb, float norm_eps,
                                     T* __restrict__ normed, int H,
                                     const int* __restrict__ pos_of_pair,
                                     const float* __restrict__ pair_w, int top) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const size_t src = (size_t)(rows ? rows[r] : r) * H, dst = (size_t)r * H;
  float yinv = 1.f;
  if (ymode != 0) {
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
      float v;
      if (top > 0) {                         // y[pair rows]: the token's pairs added up in order
        v = 0.f;
        for (int k = 0; k < top; ++k) {
          const size_t pr = (src / H) * top + k;
          v = fmaf(pair_w ? pair_w[pr] : 1.f, to_f32(y[(size_t)pos_of_pair[pr] * H + j]), v);
        }
      } else {
        v = to_f32(y[src + j]);
      }
      row[j] = v;
      ss += v * v;
    }
    if (ymode == 2) {
      ss = block_sum(ss, scratch);
      yinv = 1.f / sqrtf(ss / (float)H + y_eps);
    }
  }
  float sum = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {     // a thread meets its own row[j] again
    float v = x[src + j];
    if (add_full) v += add_full[src + j];
    if (add_row) v += add_row[j];
    if (ymode == 1) v += m * (scale ? scale[j] * row[j] : row[j]);
    if (ymode == 2) v += m * (row[j] * yinv * scale[j]);
    row[j] = v;
    if (out) out[dst + j] = v;
    if (act) act[dst + j] = from_f32<T>(v);
    sum += v;
  }
  if (norm == 0) return;
  float mean = 0.f;
  if (norm == 1) mean = block_sum(sum, scratch) / (float)H;
  float sq = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float d = row[j] - mean;
    sq += d * d;
  }
  sq = block_sum(sq, scratch);
  const float sd = sqrtf(sq / (float)H + norm_eps);
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float v = (row[j] - mean) / sd * nw[j];
    if (nb) v += nb[j];
    normed[dst + j] = from_f32<T>(v);
  }
}

// The same with four channels an access and the row kept in registers (OPT quads a thread): per
// row this moves what the definition needs and nothing else.  Needs H % 4 == 0, H <= 4 * OPT *
// threads and 16-byte aligned rows.
template <typename Y, typename T, int OPT>
__global__ void stream_update_vec_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                         const Y* __restrict__ y, int ymode,
                                         const float* __restrict__ scale, float m, float y_eps,
                                         const float* __restrict__ add_full,
                                         const float* __restrict__ add_row,
                                         float* __restrict__ out, T* __restrict__ act, int norm,
                                         const float* __restrict__ nw,
                                         const float* __restrict__ nb, float norm_eps,
                                         T* __restrict__ normed, int H,
                                         const int* __restrict__ pos_of_pair,
                                         const float* __restrict__ pair_w, int top) {
  __shared__ float scratch[33];
  const int r = blockIdx.x, nq = H >> 2;
  pdl_trigger();
  pdl_wait();
  const size_t src = (size_t)(rows ? rows[r] : r) * H, dst = (size_t)r * H;
  float v[OPT][4];
  float yinv = 1.f;
  if (ymode != 0) {
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < OPT; ++u) {
      const int q = threadIdx.x + u * blockDim.x;
      if (q < nq) {
        if (top > 0) {                       // y[pair rows]: the token's pairs added up in order
#pragma unroll
          for (int i = 0; i < 4; ++i) v[u][i] = 0.f;
          for (int k = 0; k < top; ++k) {
            const size_t pr = (src / H) * top + k;
            const float pw = pair_w ? pair_w[pr] : 1.f;
            float t[4];
            Quad<Y>::load(y + (size_t)pos_of_pair[pr] * H + 4 * q, t);
#pragma unroll
            for (int i = 0; i < 4; ++i) v[u][i] = fmaf(pw, t[i], v[u][i]);
          }
        } else {
          Quad<Y>::load(y + src + 4 * q, v[u]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) ss += v[u][i] * v[u][i];
      }
    }
    if (ymode == 2) {
      ss = block_sum(ss, scratch);
      yinv = 1.f / sqrtf(ss / (float)H + y_eps);
    }
  }
  float sum = 0.f;
#pragma unroll
  for (int u = 0; u < OPT; ++u) {
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) {
      float xv[4], t[4];
      Quad<float>::load(x + src + 4 * q, xv);
      if (add_full) {
        Quad<float>::load(add_full + src + 4 * q, t);
#pragma unroll
        for (int i = 0; i < 4; ++i) xv[i] += t[i];
      }
      if (add_row) {
        Quad<float>::load(add_row + 4 * q, t);
#pragma unroll
        for (int i = 0; i < 4; ++i) xv[i] += t[i];
      }
      if (ymode != 0) {
        if (scale) Quad<float>::load(scale + 4 * q, t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (ymode == 1) xv[i] += m * (scale ? t[i] * v[u][i] : v[u][i]);
          else xv[i] += m * (v[u][i] * yinv * t[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) v[u][i] = xv[i], sum += xv[i];
      if (out) Quad<float>::store(out + dst + 4 * q, xv);
      if (act) Quad<T>::store(act + dst + 4 * q, xv);
    }
  }
  if (norm == 0) return;
  float mean = 0.f;
  if (norm == 1) mean = block_sum(sum, scratch) / (float)H;
  float sq = 0.f;
#pragma unroll
  for (int u = 0; u < OPT; ++u) {
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float d = v[u][i] - mean;
        sq += d * d;
      }
    }
  }
  sq = block_sum(sq, scratch);
  const float sd = sqrtf(sq / (float)H + norm_eps);
#pragma unroll
  for (int u = 0; u < OPT; ++u) {
    const int q = threadIdx.x + u * blockDim.x;
    if (q < nq) {
      float w[4], b[4] = {0.f, 0.f, 0.f, 0.f}, o[4];
      Quad<float>::load(nw + 4 * q, w);
      if (nb) Quad<float>::load(nb + 4 * q, b);
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = (v[u][i] - mean) / sd * w[i] + b[i];
      Quad<T>::store(normed + dst + 4 * q, o);
    }
  }
}

// One warp per (token, head); heads 0 .. nh - 1 are q heads, nh .. nh + nkv - 1 the k heads.
// qkv row: q heads from column 0, k heads from k_off, values from v_off (= k_off when the values
// are the keys as projected).  freqs[n_pairs]; pair i of a head is channels (2i, 2i + 1) if
// interleaved, else (i, i + n_pairs); channels from 2 n_pairs on pass unrotated.  qw / kw: norm
// weights of hd channels, or null for no norm.  slot_mapping null: nothing is cached.
// A factor on the queries that grows with the position: 1 + coef * ln(floor((p + 1) / every) + 1);
// every <= 0: none.
__device__ __forceinline__ float query_temperature(int p, float coef, int every) {
  return every > 0 ? 1.f + coef * logf((float)((p + 1) / every) + 1.f) : 1.f;
}

template <typename T>
__global__ void qk_norm_rope_kernel(T* __restrict__ qkv, int stride, int num_tokens, int nh,
                                    int nkv, int hd, int k_off, int v_off,
                                    const float* __restrict__ qw, const float* __restrict__ kw,
                                    float eps, float qt_coef, int qt_every,
                                    const float* __restrict__ freqs, int n_pairs,
                                    int interleaved, const int* __restrict__ positions,
                                    const int* __restrict__ slot_mapping, T* __restrict__ kpages,
                                    T* __restrict__ vpages) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();
  const int heads = nh + nkv;
  if (warp >= num_tokens * heads) return;
  const int t = warp / heads, h = warp - t * heads;
  const bool is_k = h >= nh;
  if (is_k && slot_mapping == nullptr) return;
  T* src = qkv + (size_t)t * stride + (is_k ? k_off + (h - nh) * hd : h * hd);
  const float* w = is_k ? kw : qw;
  T* dst = src;
  if (is_k) {
    const size_t slot = (size_t)slot_mapping[t];
    dst = kpages + (slot * nkv + (h - nh)) * hd;
    const T* vsrc = qkv + (size_t)t * stride + v_off + (h - nh) * hd;
    T* vdst = vpages + (slot * nkv + (h - nh)) * hd;
    for (int c = lane; c < hd; c += 32) vdst[c] = vsrc[c];
  }
  float inv = 1.f;
  if (w) {
    float ss = 0.f;
    for (int c = lane; c < hd; c += 32) {
      const float v = to_f32(src[c]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    inv = 1.f / sqrtf(ss / (float)hd + eps);
  }
  const float pos = (float)positions[t];
  const float tq = is_k ? 1.f : query_temperature(positions[t], qt_coef, qt_every);
  for (int i = lane; i < n_pairs; i += 32) {
    const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + n_pairs;
    float u = to_f32(src[a]) * inv, v = to_f32(src[b]) * inv;
    if (w) u *= w[a], v *= w[b];
    u *= tq, v *= tq;
    float sn, cs;
    sincosf(pos * freqs[i], &sn, &cs);
    dst[a] = from_f32<T>(u * cs - v * sn);
    dst[b] = from_f32<T>(v * cs + u * sn);
  }
  for (int c = 2 * n_pairs + lane; c < hd; c += 32) {
    float u = to_f32(src[c]) * inv;
    if (w) u *= w[c];
    dst[c] = from_f32<T>(u * tq);
  }
}

// The same for neighbouring pairs and heads of up to 128 channels, a multiple of 4: a block a
// token, which takes the sines and cosines of the token's angles once, into shared memory, for all
// of its heads; a warp a head at a time, a lane owns four neighbouring channels (two pairs) and
// moves them as one access.
template <typename T>
__global__ void qk_norm_rope_vec_kernel(T* __restrict__ qkv, int stride, int num_tokens, int nh,
                                        int nkv, int hd, int k_off, int v_off,
                                        const float* __restrict__ qw, const float* __restrict__ kw,
                                        float eps, float qt_coef, int qt_every,
                                        const float* __restrict__ freqs, int n_pairs,
                                        const int* __restrict__ positions,
                                        const int* __restrict__ slot_mapping,
                                        T* __restrict__ kpages, T* __restrict__ vpages) {
  extern __shared__ float tab[];                     // cos[n_pairs], sin[n_pairs]
  const int t = blockIdx.x, lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();
  {
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x)
      sincosf(pos * freqs[i], &tab[n_pairs + i], &tab[i]);
  }
  __syncthreads();
  const int heads = slot_mapping ? nh + nkv : nh;    // nothing is cached: the k heads are left
  for (int h = threadIdx.x >> 5; h < heads; h += blockDim.x >> 5) {
  const bool is_k = h >= nh;
  T* src = qkv + (size_t)t * stride + (is_k ? k_off + (h - nh) * hd : h * hd);
  const float* w = is_k ? kw : qw;
  const int c = 4 * lane;
  const bool mine = c < hd;
  T* dst = src;
  float x[4] = {0.f, 0.f, 0.f, 0.f};
  if (mine) Quad<T>::load(src + c, x);
  if (is_k) {
    const size_t slot = (size_t)slot_mapping[t];
    dst = kpages + (slot * nkv + (h - nh)) * hd;
    if (mine) {
      T* vdst = vpages + (slot * nkv + (h - nh)) * hd + c;
      if (v_off == k_off) {
        Quad<T>::store(vdst, x);                     // exact: the values are the keys as projected
      } else {
        float vv[4];
        Quad<T>::load(qkv + (size_t)t * stride + v_off + (h - nh) * hd + c, vv);
        Quad<T>::store(vdst, vv);
      }
    }
  }
  float inv = 1.f;
  if (w) {
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
    ss = warp_sum(ss);
    inv = 1.f / sqrtf(ss / (float)hd + eps);
  }
  if (!mine) continue;
  if (w) {
    float wv[4];
    Quad<float>::load(w + c, wv);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = x[i] * inv * wv[i];
  }
  if (!is_k && qt_every > 0) {
    const float tq = query_temperature(positions[t], qt_coef, qt_every);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] *= tq;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int pair = 2 * lane + i;
    if (pair < n_pairs) {
      const float cs = tab[pair], sn = tab[n_pairs + pair];
      const float u = x[2 * i], v = x[2 * i + 1];
      x[2 * i] = u * cs - v * sn;
      x[2 * i + 1] = v * cs + u * sn;
    }
  }
  Quad<T>::store(dst + c, x);
  }
}

// Eight channels a thread (hd % 8 == 0, 16-byte aligned rows).
__global__ void head_gate_vec_kernel(__nv_bfloat16* __restrict__ o,
                                     const __nv_bfloat16* __restrict__ g, int g_stride, int nh,
                                     int hd, size_t total8) {
  pdl_trigger();
  pdl_wait();
  const int row8 = nh * hd / 8, hd8 = hd / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / row8;
    const int h = (int)(i - t * row8) / hd8;
    const float s = 1.f / (1.f + expf(-to_f32(g[t * g_stride + h])));
    uint4 raw = *reinterpret_cast<const uint4*>(o + 8 * i);
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float2 a = __bfloat1622float2(p[u]);
      p[u] = __floats2bfloat162_rn(a.x * s, a.y * s);
    }
    *reinterpret_cast<uint4*>(o + 8 * i) = raw;
  }
}

template <typename T>
__global__ void head_gate_kernel(T* __restrict__ o, const T* __restrict__ g, int g_stride, int nh,
                                 int hd, size_t total) {
  pdl_trigger();
  pdl_wait();
  const int row = nh * hd;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / row;
    const int h = (int)(i - t * row) / hd;
    const float z = to_f32(g[t * g_stride + h]);
    o[i] = from_f32<T>(to_f32(o[i]) / (1.f + expf(-z)));
  }
}

__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename Z, typename T>
__global__ void token_gate_kernel(const Z* __restrict__ z, const int* __restrict__ tokens,
                                  const T* __restrict__ table, int table_stride, int off, int dim,
                                  T* __restrict__ out, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / dim;
    const int j = (int)(i - t * dim);
    const float e = to_f32(table[(size_t)tokens[t] * table_stride + off + j]);
    out[i] = from_f32<T>(gelu_tanh(to_f32(z[i])) * e);
  }
}

}  // namespace gf

using namespace gf;
using bf = __nv_bfloat16;

GF_DEFINE_PDL_SWITCH

static inline int grid_for(size_t total) {
  const size_t want = (total + 255) / 256;
  return (int)(want < 148 * 16 ? want : 148 * 16);
}

// y_dtype / act_dtype: GF_F32 or GF_BF16.  act and normed have act_dtype.
GF_EXPORT int gf_stream_update(const float* x, const int* rows, const void* y, int y_dtype,
                               int ymode, const float* scale, float m, float y_eps,
                               const float* add_full, const float* add_row, float* out, void* act,
                               int act_dtype, int norm, const float* nw, const float* nb,
                               float norm_eps, void* normed, int R, int H,
                               const int* pos_of_pair, const float* pair_w, int top,
                               void* stream) {
  if (R <= 0) return 0;
  if (top > 0 && (!pos_of_pair || ymode == 0)) return -2;
  if ((ymode != 0 && !y) || (ymode == 2 && !scale) || (norm != 0 && (!nw || !normed))) return -2;
  auto st = (cudaStream_t)stream;
  const bool aligned = (((uintptr_t)x | (uintptr_t)y | (uintptr_t)scale | (uintptr_t)add_full |
                         (uintptr_t)add_row | (uintptr_t)out | (uintptr_t)act | (uintptr_t)nw |
                         (uintptr_t)nb | (uintptr_t)normed) & 15) == 0;
  if (H % 4 == 0 && H <= 4 * 4 * 256 && aligned) {
    const int nq = H / 4;
    const dim3 vgrid(R), vblock(nq <= 128 ? 128 : 256);
#define GF_VEC(Y, T, OPT)                                                                         \
  return launch_kernel(stream_update_vec_kernel<Y, T, OPT>, vgrid, vblock, 0, st, x, rows,          \
                       (const Y*)y, ymode, scale, m, y_eps, add_full, add_row, out, (T*)act, norm,  \
                       nw, nb, norm_eps, (T*)normed, H, pos_of_pair, pair_w, top)
#define GF_OPT(Y, T)                                  \
  {                                                   \
    if (nq <= (int)vblock.x) GF_VEC(Y, T, 1);         \
    if (nq <= 2 * (int)vblock.x) GF_VEC(Y, T, 2);     \
    GF_VEC(Y, T, 4);                                  \
  }
    if (act_dtype == GF_F32) {
      if (y && y_dtype != GF_F32) return -2;
      GF_OPT(float, float)
    }
    if (y && y_dtype == GF_F32) GF_OPT(float, bf)
    GF_OPT(bf, bf)
#undef GF_OPT
#undef GF_VEC
  }
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 48 * 1024) return -4;
  const dim3 grid(R), block(H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
#define GF_GO(Y, T)                                                                             \
  return launch_kernel(stream_update_kernel<Y, T>, grid, block, smem, st, x, rows, (const Y*)y, \
                       ymode, scale, m, y_eps, add_full, add_row, out, (T*)act, norm, nw, nb,   \
                       norm_eps, (T*)normed, H, pos_of_pair, pair_w, top)
  if (act_dtype == GF_F32) {
    if (y && y_dtype != GF_F32) return -2;
    GF_GO(float, float);
  }
  if (y && y_dtype == GF_F32) GF_GO(float, bf);
  GF_GO(bf, bf);
#undef GF_GO
}

GF_EXPORT int gf_qk_norm_rope(void* qkv, int stride, int T, int nh, int nkv, int hd, int k_off,
                              int v_off, const float* qw, const float* kw, float eps,
                              float qt_coef, int qt_every,
                              const float* freqs, int n_pairs, int interleaved,
                              const int* positions, const int* slot_mapping, void* kpages,
                              void* vpages, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (2 * n_pairs > hd || (n_pairs > 0 && !freqs)) return -3;
  auto st = (cudaStream_t)stream;
  const size_t warps = (size_t)T * (nh + nkv);
  const dim3 grid((unsigned)((warps + 3) / 4)), block(128);
  const int esz = dtype == GF_F32 ? 4 : 2;
  const bool vec = (interleaved || n_pairs == 0) && hd % 4 == 0 && hd <= 128 && stride % 4 == 0 &&
                   k_off % 4 == 0 && v_off % 4 == 0 &&
                   (((uintptr_t)qkv | (uintptr_t)kpages | (uintptr_t)vpages) % (4 * esz)) == 0 &&
                   (((uintptr_t)qw | (uintptr_t)kw) & 15) == 0;
  if (vec) {
    // few tokens: a warp a head, so that no warp walks over several heads one after the other
    const int hw = nh + nkv < 16 ? nh + nkv : 16;
    const dim3 grid(T), block(T <= 256 ? 32 * hw : 128);
    const size_t smem = 2 * (size_t)n_pairs * sizeof(float);
    if (dtype == GF_F32)
      return launch_kernel(qk_norm_rope_vec_kernel<float>, grid, block, smem, st, (float*)qkv, stride,
                           T, nh, nkv, hd, k_off, v_off, qw, kw, eps, qt_coef, qt_every, freqs, n_pairs, positions,
                           slot_mapping, (float*)kpages, (float*)vpages);
    return launch_kernel(qk_norm_rope_vec_kernel<bf>, grid, block, smem, st, (bf*)qkv, stride, T, nh,
                         nkv, hd, k_off, v_off, qw, kw, eps, qt_coef, qt_every, freqs, n_pairs, positions,
                         slot_mapping, (bf*)kpages, (bf*)vpages);
  }
  if (dtype == GF_F32)
    return launch_kernel(qk_norm_rope_kernel<float>, grid, block, 0, st, (float*)qkv, stride, T,
                         nh, nkv, hd, k_off, v_off, qw, kw, eps, qt_coef, qt_every, freqs, n_pairs, interleaved,
                         positions, slot_mapping, (float*)kpages, (float*)vpages);
  return launch_kernel(qk_norm_rope_kernel<bf>, grid, block, 0, st, (bf*)qkv, stride, T, nh, nkv,
                       hd, k_off, v_off, qw, kw, eps, qt_coef, qt_every, freqs, n_pairs, interleaved, positions,
                       slot_mapping, (bf*)kpages, (bf*)vpages);
}

GF_EXPORT int gf_head_gate(void* o, const void* g, int g_stride, int T, int nh, int hd, int dtype,
                           void* stream) {
  const size_t total = (size_t)T * nh * hd;
  if (total == 0) return 0;
  auto st = (cudaStream_t)stream;
  if (dtype == GF_F32)
    return launch_kernel(head_gate_kernel<float>, dim3(grid_for(total)), dim3(256), 0, st,
                         (float*)o, (const float*)g, g_stride, nh, hd, total);
  if (hd % 8 == 0 && ((uintptr_t)o & 15) == 0)
    return launch_kernel(head_gate_vec_kernel, dim3(grid_for(total / 8)), dim3(256), 0, st, (bf*)o,
                         (const bf*)g, g_stride, nh, hd, total / 8);
  return launch_kernel(head_gate_kernel<bf>, dim3(grid_for(total)), dim3(256), 0, st, (bf*)o,
                       (const bf*)g, g_stride, nh, hd, total);
}

// z [T, dim] fp32 (z_dtype GF_F32) or of the activation type; table rows of the activation type.
GF_EXPORT int gf_token_gate(const void* z, int z_dtype, const int* tokens, const void* table,
                            int table_stride, int off, int dim, void* out, int T, int dtype,
                            void* stream) {
  const size_t total = (size_t)T * dim;
  if (total == 0) return 0;
  auto st = (cudaStream_t)stream;
  const dim3 grid(grid_for(total)), block(256);
  if (dtype == GF_F32) {
    if (z_dtype != GF_F32) return -2;
    return launch_kernel(token_gate_kernel<float, float>, grid, block, 0, st, (const float*)z,
                         tokens, (const float*)table, table_stride, off, dim, (float*)out, total);
  }
  if (z_dtype == GF_F32)
    return launch_kernel(token_gate_kernel<float, bf>, grid, block, 0, st, (const float*)z, tokens,
                         (const bf*)table, table_stride, off, dim, (bf*)out, total);
  return launch_kernel(token_gate_kernel<bf, bf>, grid, block, 0, st, (const bf*)z, tokens,
                       (const bf*)table, table_stride, off, dim, (bf*)out, total);
}
