// Latent attention: every token keeps ONE latent vector c (C channels, RMS-normed) and one rotated
// key part r (R channels) shared by all heads.  With the key up-projection folded into the query
// (q_lat = W_uk^T q_plain) a head's score against key j is (q_lat . c_j + q_rot . r_j) * scale and
// its output is sum_j p_j c_j (C channels), which the value up-projection turns into the head's
// values afterwards: multi-query attention with keys [c | r] and values c.
//
//   latent_prepare_kernel   per token: c = rmsnorm(first C of the down-projection) * w into the
//                           token's cache slot, the rotated key part into its slot, the heads'
//                           rotated query parts in fp32.  Rotation: channels (2i, 2i+1) of the first
//                           `rot` channels by the angle float(p) * freq[i], fp32.
//   latent_attention_kernel one block per (token, 8 heads), a warp a head; keys lo..p (lo = max(0,
//                           p - window + 1) with a window) visited in groups of 32 from lo, staged
//                           once per block in shared memory as fp32; running maximum, sum and the
//                           C-wide accumulator in fp32.  A row's result depends only on (lo, p) and
//                           the cache, never on how the step was cut or what else is in the batch.
#include "common.cuh"

namespace gf {

constexpr int kLatWarps = 8;        // heads per block
constexpr int kLatTile = 32;        // keys per tile (a lane a key)
constexpr int kLatMaxC = 1024;      // latent channels a lane can accumulate (32 registers)

template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ qd, int ld, int H, int D, int R, int C,
                                      int rot, const float* __restrict__ freq,
                                      const float* __restrict__ cnorm_w, float eps,
                                      const int* __restrict__ positions,
                                      const int* __restrict__ slot_mapping, T* __restrict__ c_pages,
                                      T* __restrict__ r_pages, float* __restrict__ q_rot) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const T* row = qd + (size_t)t * ld;
  const T* dkv = row + (size_t)H * (D + R);
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  const float p = (float)positions[t];
  // the latent vector
  float ss = 0.f;
  for (int j = threadIdx.x; j < C; j += blockDim.x) {
    const float v = to_f32(dkv[j]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)C + eps);
  if (slot >= 0) {
    T* cdst = c_pages + (size_t)slot * C;
    for (int j = threadIdx.x; j < C; j += blockDim.x)
      cdst[j] = from_f32<T>(to_f32(dkv[j]) / rms * cnorm_w[j]);
  }
  // rotated parts: unit u < H is a head's query part, unit H the shared key part
  const int half = rot >> 1;
  for (int i = threadIdx.x; i < (H + 1) * half; i += blockDim.x) {
    const int u = i / half, k = i - u * half;
    const T* src = u < H ? row + (size_t)u * (D + R) + D : dkv + C;
    float sn, cs;
    sincosf(p * freq[k], &sn, &cs);
    const float a = to_f32(src[2 * k]), b = to_f32(src[2 * k + 1]);
    const float lo = a * cs - b * sn, hi = b * cs + a * sn;
    if (u < H) {
      float* dst = q_rot + ((size_t)t * H + u) * R;
      dst[2 * k] = lo;
      dst[2 * k + 1] = hi;
    } else if (slot >= 0) {
      T* dst = r_pages + (size_t)slot * R;
      dst[2 * k] = from_f32<T>(lo);
      dst[2 * k + 1] = from_f32<T>(hi);
    }
  }
  const int tail = R - rot;                       // channels that pass unrotated
  for (int i = threadIdx.x; i < (H + 1) * tail; i += blockDim.x) {
    const int u = i / tail, k = rot + (i - u * tail);
    if (u < H)
      q_rot[((size_t)t * H + u) * R + k] = to_f32(row[(size_t)u * (D + R) + D + k]);
    else if (slot >= 0)
      r_pages[(size_t)slot * R + k] = dkv[C + k];
  }
}

// A token's two latent vectors out of one projection row: the query latent (Q channels from q_col,
// RMS-normed with qw into cq, in the activation type, for the query up-projection) and the key/value
// latent (C channels from c_col, RMS-normed with cw into the token's cache slot).  Either may be
// absent (Q = 0; slot_mapping null).  One block a token.
// Two channels an access: a pair of T as two floats, and back.
__device__ __forceinline__ float2 load_pair(const float* p) {
  return *reinterpret_cast<const float2*>(p);
}
__device__ __forceinline__ float2 load_pair(const bf16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void store_pair(float* p, float a, float b) {
  *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
__device__ __forceinline__ void store_pair(bf16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// PAIRS: every column offset and count is even and the rows are aligned for pairs.  The two sums
// of squares are reduced together (one pass of barriers for both norms).
template <typename T, bool PAIRS>
__global__ void latent_norms_kernel(const T* __restrict__ proj, int ld, int q_col, int Q,
                                    const float* __restrict__ qw, T* __restrict__ cq, int c_col,
                                    int C, const float* __restrict__ cw, float eps,
                                    const int* __restrict__ slot_mapping, T* __restrict__ c_pages) {
  __shared__ float scratch[2][33];
  const int t = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const T* row = proj + (size_t)t * ld;
  const bool write_c = slot_mapping != nullptr && C > 0;
  const int Cn = write_c ? C : 0;
  constexpr int W = PAIRS ? 2 : 1;
  float ssq = 0.f, ssc = 0.f;
  for (int j = threadIdx.x * W; j < Q; j += blockDim.x * W) {
    if (PAIRS) {
      const float2 v = load_pair(row + q_col + j);
      ssq += v.x * v.x + v.y * v.y;
    } else {
      const float v = to_f32(row[q_col + j]);
      ssq += v * v;
    }
  }
  for (int j = threadIdx.x * W; j < Cn; j += blockDim.x * W) {
    if (PAIRS) {
      const float2 v = load_pair(row + c_col + j);
      ssc += v.x * v.x + v.y * v.y;
    } else {
      const float v = to_f32(row[c_col + j]);
      ssc += v * v;
    }
  }
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    ssq = warp_sum(ssq);
    ssc = warp_sum(ssc);
    if (lane == 0) scratch[0][warp] = ssq, scratch[1][warp] = ssc;
    __syncthreads();
    if (warp < 2) {
      float v = lane < nwarps ? scratch[warp][lane] : 0.f;
      v = warp_sum(v);
      if (lane == 0) scratch[warp][32] = v;
    }
    __syncthreads();
    ssq = scratch[0][32];
    ssc = scratch[1][32];
  }
  if (Q > 0) {
    const float inv = 1.f / sqrtf(ssq / (float)Q + eps);
    T* dst = cq + (size_t)t * Q;
    for (int j = threadIdx.x * W; j < Q; j += blockDim.x * W) {
      if (PAIRS) {
        const float2 v = load_pair(row + q_col + j);
        store_pair(dst + j, v.x * inv * qw[j], v.y * inv * qw[j + 1]);
      } else {
        dst[j] = from_f32<T>(to_f32(row[q_col + j]) * inv * qw[j]);
      }
    }
  }
  if (write_c) {
    const float inv = 1.f / sqrtf(ssc / (float)C + eps);
    T* dst = c_pages + (size_t)slot_mapping[t] * C;
    for (int j = threadIdx.x * W; j < C; j += blockDim.x * W) {
      if (PAIRS) {
        const float2 v = load_pair(row + c_col + j);
        store_pair(dst + j, v.x * inv * cw[j], v.y * inv * cw[j + 1]);
      } else {
        dst[j] = from_f32<T>(to_f32(row[c_col + j]) * inv * cw[j]);
      }
    }
  }
}

// The latent vectors of the step's requests side by side: row (b W + j) page + r of `out` is row r
// of the page that request b's block table names at j (clamped to the pool: what lies behind a
// request's last page is copied from somewhere and never read as a key).  `own[b W + j] = b W + j`
// is the block table under which `out`, seen as B W pages, is a cache of its own.  One block a
// row; 16 bytes an access where rows allow (`vec`).
__global__ void latent_gather_kernel(const unsigned char* __restrict__ c_pages,
                                     const int* __restrict__ table, int table_stride, int W,
                                     int page, int row_bytes, int num_pages, int vec,
                                     unsigned char* __restrict__ out, int* __restrict__ own) {
  const int row = blockIdx.x;
  const int lp = row / page, r = row - lp * page;         // lp = b W + j
  const int b = lp / W, j = lp - b * W;
  pdl_trigger();
  pdl_wait();
  int pg = table[(size_t)b * table_stride + j];
  pg = pg < 0 ? 0 : (pg >= num_pages ? num_pages - 1 : pg);
  const unsigned char* src = c_pages + ((size_t)pg * page + r) * row_bytes;
  unsigned char* dst = out + (size_t)row * row_bytes;
  if (vec) {
    for (int i = threadIdx.x * 16; i < row_bytes; i += blockDim.x * 16)
      *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
  } else {
    for (int i = threadIdx.x * 2; i < row_bytes; i += blockDim.x * 2)
      *reinterpret_cast<unsigned short*>(dst + i) = *reinterpret_cast<const unsigned short*>(src + i);
  }
  if (r == 0 && threadIdx.x == 0) own[lp] = lp;
}

template <typename T>
__global__ void latent_attention_kernel(const float* __restrict__ q_lat,   // [H, T, C]
                                        const float* __restrict__ q_rot,   // [T, H, R]
                                        const T* __restrict__ c_pages, const T* __restrict__ r_pages,
                                        const int* __restrict__ block_table, int table_stride,
                                        const int* __restrict__ seq_of_token,
                                        const int* __restrict__ positions, T* __restrict__ out,
                                        int num_tokens, int H, int C, int R, int page_size,
                                        int window, float scale) {
  extern __shared__ float smem[];
  const int Dk = C + R, ks = Dk + 1;               // odd stride: a lane a key without conflicts
  float* keys = smem;                              // [kLatTile][ks]
  float* qs = smem + kLatTile * ks;                // [kLatWarps][Dk]
  __shared__ int slots[kLatTile];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * kLatWarps + warp;
  const bool live = h < H;
  pdl_trigger();
  pdl_wait();
  const int b = seq_of_token[t];
  const int p = positions[t];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int* tbl = block_table + (size_t)b * table_stride;
  if (live) {
    const float* ql = q_lat + ((size_t)h * num_tokens + t) * C;
    const float* qr = q_rot + ((size_t)t * H + h) * R;
    float* q = qs + warp * Dk;
    for (int d = lane; d < C; d += 32) q[d] = ql[d];
    for (int d = lane; d < R; d += 32) q[C + d] = qr[d];
  }
  float acc[kLatMaxC / 32];
#pragma unroll
  for (int i = 0; i < kLatMaxC / 32; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int c0 = lo; c0 <= p; c0 += kLatTile) {
    const int nvalid = min(kLatTile, p - c0 + 1);
    __syncthreads();                               // the tile before is no longer read
    if (threadIdx.x < kLatTile) {
      const int c = c0 + threadIdx.x;
      slots[threadIdx.x] = c <= p ? tbl[c / page_size] * page_size + c % page_size : 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nvalid * Dk; i += blockDim.x) {
      const int j = i / Dk, d = i - j * Dk;
      const size_t s = (size_t)slots[j];
      keys[j * ks + d] = d < C ? to_f32(c_pages[s * C + d]) : to_f32(r_pages[s * R + (d - C)]);
    }
    __syncthreads();
    if (live) {
      const float* q = qs + warp * Dk;
      const bool valid = lane < nvalid;
      float s = -INFINITY;
      if (valid) {
        const float* k = keys + lane * ks;
        float dot = 0.f;
        for (int d = 0; d < Dk; ++d) dot = fmaf(q[d], k[d], dot);
        s = dot * scale;
      }
      const float m_new = fmaxf(m, warp_max(s));
      const float pexp = valid ? expf(s - m_new) : 0.f;
      const float corr = expf(m - m_new);
      l = l * corr + warp_sum(pexp);
#pragma unroll
      for (int i = 0; i < kLatMaxC / 32; ++i) acc[i] *= corr;
      for (int j = 0; j < nvalid; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pexp, j);
        const float* v = keys + j * ks;
#pragma unroll
        for (int i = 0; i < kLatMaxC / 32; ++i) {
          const int d = lane + 32 * i;
          if (d < C) acc[i] = fmaf(pj, v[d], acc[i]);
        }
      }
      m = m_new;
    }
  }
  if (live) {
    T* o = out + ((size_t)h * num_tokens + t) * C;
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < kLatMaxC / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < C) o[d] = from_f32<T>(acc[i] * inv);
    }
  }
}


// ---- the same attention on the tensor cores (bf16 cache) ----------------------------------------
// A block = one token x 16 heads (the rows of an m16n8k16 tile), sixteen warps.  Keys come in tiles
// of 64 through two stages of shared memory (16-byte cp.async straight from the pages, rows past the
// token's position zero-filled).  Scores: warp w takes keys 8 (w % 8) .. + 7 of the tile over one
// half (w / 8) of the reduction [c | r] (two accumulators, even and odd k-steps, so that the
// products do not wait for one another); the halves and then the row maxima meet in shared memory;
// P goes to shared memory as bf16 and every warp multiplies it with its share of the latent
// channels, read from the SAME tile (the values are the first C channels of the keys) through
// transposing ldmatrix loads.  With one block of this size an SM (its shared memory holds the two
// key stages) the sixteen warps are what hides the latencies of the chain.  Running maximum, sums and
// the output accumulator are fp32; the query is rounded to bf16 once.
// Needs C % 16 == 0, R % 16 == 0, C <= 128 * NT (NT column tiles of 8 a warp).  Few tokens with many
// keys (decode steps of small batches): several blocks share a token's tiles (blockIdx.z) and a
// second kernel merges their sums, as the decode kernel of the grouped-query attention does.
constexpr int kMmaTile = 64;
constexpr int kMmaWarps = 16;

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n)
               : "memory");
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
               : "=r"(r[0]), "=r"(r[1])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
               : "=r"(r[0]), "=r"(r[1])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int NT>
__global__ void __launch_bounds__(kMmaWarps * 32)
latent_attention_mma_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot,
                            const bf16* __restrict__ c_pages, const bf16* __restrict__ r_pages,
                            const int* __restrict__ block_table, int table_stride,
                            const int* __restrict__ seq_of_token,
                            const int* __restrict__ positions, bf16* __restrict__ out,
                            int num_tokens, int H, int C, int R, int page_size, int window,
                            float scale, int nsplit, float* __restrict__ part_o,
                            float* __restrict__ part_ml) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int Dk = C + R, ld = Dk + 8;
  constexpr int pld = kMmaTile + 8;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);              // [16][ld]
  bf16* Ks = Qs + 16 * ld;                                   // [2][64][ld]
  bf16* Ps = Ks + 2 * kMmaTile * ld;                         // [16][pld]
  float* red = reinterpret_cast<float*>(Ps + 16 * pld);      // [8][16]
  float* sred = red + 8 * 16;                                // [2][16][64]: the halves' scores
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int t = blockIdx.x, h0 = blockIdx.y * 16;
  pdl_trigger();
  pdl_wait();
  const int b = seq_of_token[t];
  const int p = positions[t];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int* tbl = block_table + (size_t)b * table_stride;
  for (int i = threadIdx.x; i < 16 * Dk; i += blockDim.x) {
    const int r = i / Dk, d = i - r * Dk, h = h0 + r;
    float v = 0.f;
    if (h < H) v = d < C ? q_lat[((size_t)h * num_tokens + t) * C + d]
                         : q_rot[((size_t)t * H + h) * R + (d - C)];
    Qs[r * ld + d] = __float2bfloat16_rn(v);
  }
  const int nchunk = Dk >> 3;
  // The page of this thread's key in a tile is looked up a tile ahead of the copies that need it,
  // so that no tile waits for the table.
  const int kj = threadIdx.x >> 3;                           // eight threads a key
  auto page_of = [&](int tile) {
    const int c = lo + tile * kMmaTile + kj;
    return c <= p ? tbl[c / page_size] : -1;
  };
  auto ask = [&](int tile, int page) {
    bf16* dst = Ks + (size_t)(tile & 1) * kMmaTile * ld;
    const int c = lo + tile * kMmaTile + kj;
    const bool ok = page >= 0;
    const size_t slot = ok ? (size_t)page * page_size + c % page_size : 0;
    for (int i = threadIdx.x & 7; i < nchunk; i += 8) {
      const int d = i << 3;
      const bf16* src = d < C ? c_pages + slot * C + d : r_pages + slot * R + (d - C);
      cp_async_16(dst + (size_t)kj * ld + d, src, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // nsplit > 1 (few tokens with many keys): block z of a token takes a share of its tiles and
  // leaves its unnormalised sums, which latent_merge_kernel puts together
  const int all_tiles = (p - lo) / kMmaTile + 1;
  const int share = (all_tiles + nsplit - 1) / nsplit;
  const int tile0 = (int)blockIdx.z * share;
  const int ntiles = min(all_tiles, tile0 + share);
  const int ctiles = C >> 3;                                 // column tiles of 8 in all
  const int ntw = (ctiles + kMmaWarps - 1) / kMmaWarps;      // of which this warp owns up to ntw
  float o[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, lsum[2] = {0.f, 0.f};
  // ldmatrix addresses: A (16 rows x 16 k): lanes 0-15 rows, lanes 16-31 the second 8 k;
  // B of the scores (8 keys x 16 k): lanes 0-7 keys at k, lanes 8-15 the same keys at k + 8
  const int a_row = lane & 15, a_col = (lane >> 4) << 3;
  const int kg = warp & 7, half = warp >> 3;                 // this warp's keys and k half
  const int b_row = 8 * kg + (lane & 7), b_col = ((lane >> 3) & 1) << 3;
  const int k_mid = ((Dk >> 4) >> 1) << 4;                   // the first half's channels
  const int k_lo = half ? k_mid : 0, k_hi = half ? Dk : k_mid;
  if (tile0 < ntiles) ask(tile0, page_of(tile0));
  int page_next = tile0 + 1 < ntiles ? page_of(tile0 + 1) : -1;
  for (int it = tile0; it < ntiles; ++it) {
    if (it + 1 < ntiles) {
      ask(it + 1, page_next);
      page_next = it + 2 < ntiles ? page_of(it + 2) : -1;
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const bf16* K = Ks + (size_t)(it & 1) * kMmaTile * ld;
    // ---- scores of this warp's 8 keys
    float s0[4] = {}, s1[4] = {};
    const bf16* qa = Qs + a_row * ld + a_col;
    const bf16* kb = K + (size_t)b_row * ld + b_col;
    int kk = k_lo;
#pragma unroll 2
    for (; kk + 32 <= k_hi; kk += 32) {
      uint32_t a0[4], a1[4], b0[2], b1[2];
      ldsm_x4(a0, qa + kk);
      ldsm_x2(b0, kb + kk);
      ldsm_x4(a1, qa + kk + 16);
      ldsm_x2(b1, kb + kk + 16);
      mma_bf16(s0, a0, b0);
      mma_bf16(s1, a1, b1);
    }
    if (kk < k_hi) {
      uint32_t a0[4], b0[2];
      ldsm_x4(a0, qa + kk);
      ldsm_x2(b0, kb + kk);
      mma_bf16(s0, a0, b0);
    }
    {                                              // the halves meet
      float* mine = sred + half * 16 * kMmaTile + 8 * kg + 2 * t4;
      *reinterpret_cast<float2*>(mine + g * kMmaTile) = make_float2(s0[0] + s1[0], s0[1] + s1[1]);
      *reinterpret_cast<float2*>(mine + (g + 8) * kMmaTile) = make_float2(s0[2] + s1[2], s0[3] + s1[3]);
    }
    __syncthreads();
    float s[4];
    {
      const float* at = sred + 8 * kg + 2 * t4;
      const float2 u0 = *reinterpret_cast<const float2*>(at + g * kMmaTile);
      const float2 u1 = *reinterpret_cast<const float2*>(at + 16 * kMmaTile + g * kMmaTile);
      const float2 w0 = *reinterpret_cast<const float2*>(at + (g + 8) * kMmaTile);
      const float2 w1 = *reinterpret_cast<const float2*>(at + 16 * kMmaTile + (g + 8) * kMmaTile);
      s[0] = u0.x + u1.x, s[1] = u0.y + u1.y, s[2] = w0.x + w1.x, s[3] = w0.y + w1.y;
    }
    const int key0 = lo + it * kMmaTile + 8 * kg + 2 * t4;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      s[e] = key0 + (e & 1) <= p ? s[e] * scale : -INFINITY;
      mx[e >> 1] = fmaxf(mx[e >> 1], s[e]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      if (t4 == 0 && half == 0) red[kg * 16 + g + 8 * r] = mx[r];
    }
    __syncthreads();
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      float mt = red[row];
#pragma unroll
      for (int w = 1; w < 8; ++w) mt = fmaxf(mt, red[w * 16 + row]);
      const float mn = fmaxf(m[r], mt);
      corr[r] = expf(m[r] - mn);
      m[r] = mn;
      lsum[r] *= corr[r];
    }
    {
      const float p0 = expf(s[0] - m[0]), p1 = expf(s[1] - m[0]);
      const float p2 = expf(s[2] - m[1]), p3 = expf(s[3] - m[1]);
      lsum[0] += p0 + p1;
      lsum[1] += p2 + p3;
      const int col = 8 * kg + 2 * t4;
      if (half == 0) {
        *reinterpret_cast<uint32_t*>(Ps + g * pld + col) = pack_bf16(p0, p1);
        *reinterpret_cast<uint32_t*>(Ps + (g + 8) * pld + col) = pack_bf16(p2, p3);
      }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      o[j][0] *= corr[0], o[j][1] *= corr[0];
      o[j][2] *= corr[1], o[j][3] *= corr[1];
    }
    __syncthreads();
    // ---- this warp's share of the latent channels
#pragma unroll
    for (int ks = 0; ks < kMmaTile; ks += 16) {
      uint32_t a[4];
      ldsm_x4(a, Ps + a_row * pld + ks + a_col);
      const bf16* vrow = K + (size_t)(ks + (lane & 15)) * ld;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int ct = warp * ntw + j;
        if (j < ntw && ct < ctiles) {
          uint32_t bb[2];
          ldsm_x2_trans(bb, vrow + ct * 8);
          mma_bf16(o[j], a, bb);
        }
      }
    }
    __syncthreads();                               // the stage and P are free again
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    lsum[r] += __shfl_xor_sync(0xffffffffu, lsum[r], 1);
    lsum[r] += __shfl_xor_sync(0xffffffffu, lsum[r], 2);
    if (t4 == 0 && half == 0) red[kg * 16 + g + 8 * r] = lsum[r];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r, h = h0 + row;
    if (h >= H) continue;
    float l = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) l += red[w * 16 + row];
    if (nsplit > 1) {
      const size_t at = ((size_t)blockIdx.z * num_tokens + t) * H + h;
      if (warp == 0 && t4 == 0) part_ml[2 * at] = m[r], part_ml[2 * at + 1] = l;
      float* dst = part_o + at * C;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int ct = warp * ntw + j;
        if (j < ntw && ct < ctiles)
          *reinterpret_cast<float2*>(dst + ct * 8 + 2 * t4) = make_float2(o[j][2 * r], o[j][2 * r + 1]);
      }
      continue;
    }
    const float inv = 1.f / l;
    bf16* dst = out + ((size_t)h * num_tokens + t) * C;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int ct = warp * ntw + j;
      if (j < ntw && ct < ctiles)
        *reinterpret_cast<uint32_t*>(dst + ct * 8 + 2 * t4) =
            pack_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
    }
  }
}

// out[h, t, :] = sum_z o_z exp(m_z - M) / sum_z l_z exp(m_z - M): a warp a (token, head).
__global__ void latent_merge_kernel(const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml, bf16* __restrict__ out,
                                    int num_tokens, int H, int C, int nsplit) {
  const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();
  if (pair >= num_tokens * H) return;
  const int t = pair / H, h = pair - t * H;
  constexpr int kMaxSplits = 16;
  float w[kMaxSplits];                             // a share's weight exp(m_z - M), 0 if empty
  float M = -INFINITY, L = 0.f;
#pragma unroll
  for (int z = 0; z < kMaxSplits; ++z) {
    w[z] = z < nsplit ? part_ml[2 * (((size_t)z * num_tokens + t) * H + h)] : -INFINITY;
    M = fmaxf(M, w[z]);
  }
#pragma unroll
  for (int z = 0; z < kMaxSplits; ++z) {
    const float lz = z < nsplit ? part_ml[2 * (((size_t)z * num_tokens + t) * H + h) + 1] : 0.f;
    w[z] = lz > 0.f ? expf(w[z] - M) : 0.f;
    L += lz * w[z];
  }
  const float inv = 1.f / L;
  bf16* dst = out + ((size_t)h * num_tokens + t) * C;
  const size_t step = (size_t)num_tokens * H * C;
  const float* src = part_o + ((size_t)t * H + h) * C;
  for (int c = lane; c < C; c += 32) {
    float acc = 0.f;
#pragma unroll
    for (int z = 0; z < kMaxSplits; ++z)
      if (z < nsplit && w[z] > 0.f) acc = fmaf(src[z * step + c], w[z], acc);
    dst[c] = __float2bfloat16_rn(acc * inv);
  }
}

}  // namespace gf

using namespace gf;
using bf = __nv_bfloat16;

GF_DEFINE_PDL_SWITCH

GF_EXPORT int gf_latent_prepare(const void* qd, int ld, int H, int D, int R, int C, int rot,
                                const float* freq, const float* cnorm_w, float eps,
                                const int* positions, const int* slot_mapping, void* c_pages,
                                void* r_pages, float* q_rot, int T, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (rot % 2 || rot > R) return -3;
  auto st = (cudaStream_t)stream;
  if (dtype == GF_F32)
    return launch_kernel(latent_prepare_kernel<float>, dim3(T), dim3(128), 0, st, (const float*)qd,
                         ld, H, D, R, C, rot, freq, cnorm_w, eps, positions, slot_mapping,
                         (float*)c_pages, (float*)r_pages, q_rot);
  return launch_kernel(latent_prepare_kernel<bf>, dim3(T), dim3(128), 0, st, (const bf*)qd, ld, H,
                       D, R, C, rot, freq, cnorm_w, eps, positions, slot_mapping, (bf*)c_pages,
                       (bf*)r_pages, q_rot);
}

GF_EXPORT int gf_latent_norms(const void* proj, int ld, int q_col, int Q, const float* qw, void* cq,
                              int c_col, int C, const float* cw, float eps,
                              const int* slot_mapping, void* c_pages, int T, int dtype,
                              void* stream) {
  if (T <= 0) return 0;
  auto st = (cudaStream_t)stream;
  const int widest = Q > C ? Q : C;
  const dim3 grid(T), block(widest > 512 ? 256 : 128);
  const size_t esz = dtype == GF_F32 ? 4 : 2;
  const bool pairs = !((ld | q_col | Q | c_col | C) & 1) && (uintptr_t)proj % (2 * esz) == 0 &&
                     (uintptr_t)cq % (2 * esz) == 0 && (uintptr_t)c_pages % (2 * esz) == 0;
#define GF_NORMS(TT, P)                                                                        \
  return launch_kernel(latent_norms_kernel<TT, P>, grid, block, 0, st, (const TT*)proj, ld,     \
                       q_col, Q, qw, (TT*)cq, c_col, C, cw, eps, slot_mapping, (TT*)c_pages)
  if (dtype == GF_F32) {
    if (pairs) GF_NORMS(float, true);
    GF_NORMS(float, false);
  }
  if (pairs) GF_NORMS(bf, true);
  GF_NORMS(bf, false);
#undef GF_NORMS
}

// c_pages [num_pages, page, C] (elements of `elem_bytes`: 2 or 4), table [B, table_stride] ->
// out [B W page, C], own [B W].
GF_EXPORT int gf_latent_gather(const void* c_pages, const int* table, int table_stride, int B,
                               int W, int page, int C, int elem_bytes, int num_pages, void* out,
                               int* own, void* stream) {
  if (B <= 0 || W <= 0) return 0;
  if (page <= 0 || C <= 0 || num_pages <= 0 || (elem_bytes != 2 && elem_bytes != 4)) return -3;
  const long long rows = (long long)B * W * page;
  if (rows >= (1ll << 31)) return -3;
  const int row_bytes = C * elem_bytes;
  const int vec = row_bytes % 16 == 0 && (uintptr_t)c_pages % 16 == 0 && (uintptr_t)out % 16 == 0;
  return launch_kernel(latent_gather_kernel, dim3((unsigned)rows), dim3(row_bytes >= 1024 ? 64 : 32),
                       0, (cudaStream_t)stream, (const unsigned char*)c_pages, table, table_stride,
                       W, page, row_bytes, num_pages, vec, (unsigned char*)out, own);
}

GF_EXPORT int gf_latent_attention(const float* q_lat, const float* q_rot, const void* c_pages,
                                  const void* r_pages, const int* block_table, int table_stride,
                                  const int* seq_of_token, const int* positions, void* out, int T,
                                  int H, int C, int R, int page_size, int window, float scale,
                                  int dtype, int nsplit, float* part_o, float* part_ml,
                                  void* stream) {
  if (T <= 0) return 0;
  if (C > kLatMaxC || C <= 0 || R < 0) return -3;
  const int Dk = C + R;
  if (dtype == GF_BF16 && C % 16 == 0 && R % 16 == 0 && (uintptr_t)c_pages % 16 == 0 &&
      (uintptr_t)r_pages % 16 == 0) {
    const int ld = Dk + 8;
    const size_t bytes = ((size_t)16 * ld + (size_t)2 * kMmaTile * ld + 16 * (kMmaTile + 8)) * 2 +
                         (8 * 16 + 2 * 16 * kMmaTile) * sizeof(float);
    if (bytes <= 220 * 1024) {
      static OncePerDevice once_mma;
      const int rc = once_mma.run([] {
        cudaError_t e = cudaSuccess;
#define GF_ATTR(NT)                                                                         \
  if (e == cudaSuccess)                                                                     \
    e = cudaFuncSetAttribute(latent_attention_mma_kernel<NT>,                               \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        GF_ATTR(1) GF_ATTR(2) GF_ATTR(4)
#undef GF_ATTR
        return e;
      });
      if (rc) return rc;
      if (nsplit < 1 || nsplit > 16 || (nsplit > 1 && (!part_o || !part_ml))) nsplit = 1;
      const dim3 grid(T, (H + 15) / 16, nsplit), block(kMmaWarps * 32);
      auto st = (cudaStream_t)stream;
      int rc2 = -3;
#define GF_GO(NT)                                                                              \
  if (rc2 == -3 && C <= 128 * NT)                                                              \
    rc2 = launch_kernel(latent_attention_mma_kernel<NT>, grid, block, bytes, st, q_lat, q_rot,  \
                        (const bf*)c_pages, (const bf*)r_pages, block_table, table_stride,      \
                        seq_of_token, positions, (bf*)out, T, H, C, R, page_size, window, scale, \
                        nsplit, part_o, part_ml)
      GF_GO(1);
      GF_GO(2);
      GF_GO(4);
#undef GF_GO
      if (rc2 || nsplit == 1) return rc2;
      return launch_kernel(latent_merge_kernel, dim3((T * H + 3) / 4), dim3(128), 0, st,
                           (const float*)part_o, (const float*)part_ml, (bf*)out, T, H, C, nsplit);
    }
  }
  const size_t smem = ((size_t)kLatTile * (Dk + 1) + (size_t)kLatWarps * Dk) * sizeof(float);
  if (smem > 200 * 1024) return -3;
  auto st = (cudaStream_t)stream;
  const dim3 grid(T, (H + kLatWarps - 1) / kLatWarps), block(kLatWarps * 32);
  static OncePerDevice once;
  const int rc = once.run([] {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<float>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(latent_attention_kernel<bf>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  });
  if (rc) return rc;
  if (dtype == GF_F32)
    return launch_kernel(latent_attention_kernel<float>, grid, block, smem, st, q_lat, q_rot,
                         (const float*)c_pages, (const float*)r_pages, block_table, table_stride,
                         seq_of_token, positions, (float*)out, T, H, C, R, page_size, window,
                         scale);
  return launch_kernel(latent_attention_kernel<bf>, grid, block, smem, st, q_lat, q_rot,
                       (const bf*)c_pages, (const bf*)r_pages, block_table, table_stride,
                       seq_of_token, positions, (bf*)out, T, H, C, R, page_size, window, scale);
}
