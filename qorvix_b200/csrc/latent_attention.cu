// Attention over a paged cache of low-rank latents (one row per token: the normed latent c of `rank`
// entries followed by one rotated key part of `dr` entries that all heads share).
//
// Per head h the unrotated key of token j is Wuk_h c_j and its value Wuv_h c_j.  Neither is ever formed:
//   score(t, j) = (q_plain . Wuk_h c_j + q_rot . kr_j) * scale = ((Wuk_h^T q_plain) . c_j + q_rot . kr_j) * scale
//   out(t)      = Wuv_h (sum_j p_j c_j)
// so a query is first carried into the latent space (rank entries), attention then runs as if all heads
// shared one key/value head whose key row is [c | kr] and whose value row is c, and the head's value
// matrix is applied to the weighted latent afterwards.  A sigmoid gate multiplies the output.
//
// qv_latent_prepare: per token, RMS norm of the latent part of the down projection, interleaved-pair
//   rotation of the shared key part, write of both into the token's cache row; rotation of every head's
//   query part in place.
// qv_latent_attention_generic: one warp per (token, head), float32 arithmetic whatever the storage type,
//   keys in blocks of 32 aligned to absolute positions with a running maximum and sum, so a position's
//   result depends on the position and the cache only.  Serves the true 32-bit path and every size.
#include "common.cuh"

// proj[t] = [... q: H * (dn + dr) at q_off ... down: rank + dr at kv_off ...], row stride ld.
// Rotation: entries (2i, 2i+1) of the first `rot` entries of a rotated part, angle row tok_pos of cos_sin.
template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(
    T* __restrict__ proj, int ld, int q_off, int kv_off, T* __restrict__ cache, const float* __restrict__ norm_w, float eps,
    const float2* __restrict__ cos_sin, int table_rows, const int* __restrict__ tok_pos, const int* __restrict__ tok_seg,
    const int* __restrict__ block_table, int max_blocks, int H, int dn, int dr, int rank, int rot, int page) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  T* row = proj + (size_t)t * ld;
  const float2* cs = cos_sin + (size_t)(pos < table_rows ? pos : table_rows - 1) * (rot >> 1);
  const int pg = block_table[(size_t)tok_seg[t] * max_blocks + pos / page];
  T* dst = cache + ((size_t)pg * page + (size_t)(pos % page)) * (rank + dr);
  // the latent: x * rsqrt(mean(x^2) + eps) * w
  const T* lat = row + kv_off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_f(lat[i]); ss += v * v; }
  const float total = block_sum(ss, red);
  const float sc = 1.0f / sqrtf(total / (float)rank + eps);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f<T>(to_f(lat[i]) * sc * norm_w[i]);
  // the shared rotated key part
  const T* kr = lat + rank;
  for (int i = threadIdx.x; i < dr; i += blockDim.x) {
    float v = to_f(kr[i]);
    if (i < rot) {
      const float2 c = cs[i >> 1];
      const float other = to_f(kr[i ^ 1]);
      v = (i & 1) ? v * c.x + other * c.y : v * c.x - other * c.y;
    }
    dst[rank + i] = from_f<T>(v);
  }
  // every head's rotated query part, in place (a pair is handled by one thread)
  const int pairs = rot >> 1;
  for (int k = threadIdx.x; k < H * pairs; k += blockDim.x) {
    const int h = k / pairs, i = k - h * pairs;
    T* qr = row + q_off + (size_t)h * (dn + dr) + dn + 2 * i;
    const float a = to_f(qr[0]), b = to_f(qr[1]);
    const float2 c = cs[i];
    qr[0] = from_f<T>(a * c.x - b * c.y);
    qr[1] = from_f<T>(b * c.x + a * c.y);
  }
}

extern "C" int qv_latent_prepare(void* proj, int ld, int q_off, int kv_off, void* cache, const float* norm_w, float eps,
                                 const float* cos_sin, int table_rows, const int* tok_pos, const int* tok_seg,
                                 const int* block_table, int max_blocks, int T, int H, int dn, int dr, int rank, int rot,
                                 int page, int dt, void* stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > dr || (rot & 1) || rank <= 0) return QV_ERR_UNSUPPORTED;
  QV_DISPATCH_DT(dt, TT,
                 return qv_launch(latent_prepare_kernel<TT>, dim3(T), dim3(256), 0, (cudaStream_t)stream, (TT*)proj, ld, q_off, kv_off,
                                  (TT*)cache, norm_w, eps, (const float2*)cos_sin, table_rows, tok_pos, tok_seg, block_table,
                                  max_blocks, H, dn, dr, rank, rot, page));
  return QV_ERR_UNSUPPORTED;
}

#define LAT_MAX_RANK 1024

// q: rows of [dn unrotated | dr rotated] per head at q (row stride ld_q); wuk [H * dn, rank]; wuv [H * dv, rank];
// gate (may be null) and out: [T, H * dv] with their row strides.
template <typename T, typename TW>
__global__ void __launch_bounds__(128) latent_attention_generic_kernel(
    T* __restrict__ out, int ld_out, const T* __restrict__ q, int ld_q, const T* __restrict__ gate, int ld_gate,
    const T* __restrict__ cache, const TW* __restrict__ wuk, const TW* __restrict__ wuv, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_seg, const int* __restrict__ block_table, int max_blocks, int H, int dn, int dr, int dv,
    int rank, int page, int window, float scale) {
  extern __shared__ float sm_all[];              // 4 warps x (rank + dr + dn) floats
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x * 4 + warp;
  const int t = blockIdx.y;
  if (h >= H) return;
  const int kw = rank + dr;
  float* qs = sm_all + (size_t)warp * (kw + dn);   // [rank latent query | dr rotated query]
  float* qp = qs + kw;                             // dn unrotated query entries
  const T* qrow = q + (size_t)t * ld_q + (size_t)h * (dn + dr);
  for (int i = lane; i < dn; i += 32) qp[i] = to_f(qrow[i]);
  for (int i = lane; i < dr; i += 32) qs[rank + i] = to_f(qrow[dn + i]);
  __syncwarp();
  // the query in the latent space: qs[r] = sum_i q_plain[i] * wuk[h * dn + i][r]
  for (int r = lane; r < rank; r += 32) {
    float acc = 0.f;
    for (int i = 0; i < dn; ++i) acc = fmaf(qp[i], to_f(wuk[((size_t)h * dn + i) * rank + r]), acc);
    qs[r] = acc;
  }
  __syncwarp();

  const int pos = tok_pos[t];
  const int* bt = block_table + (size_t)tok_seg[t] * max_blocks;
  const int lo = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
  constexpr int NREG = LAT_MAX_RANK / 32;
  float o[NREG];
#pragma unroll
  for (int j = 0; j < NREG; ++j) o[j] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int kb = (lo >> 5) << 5; kb <= pos; kb += 32) {
    const int tk = kb + lane;
    const bool valid = tk >= lo && tk <= pos;
    size_t base = 0;
    float s = -INFINITY;
    if (valid) {
      base = ((size_t)bt[tk / page] * page + (size_t)(tk % page)) * kw;
      const T* kp = cache + base;
      float dot = 0.f;
      for (int i = 0; i < kw; ++i) dot = fmaf(qs[i], to_f(kp[i]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int j = 0; j < NREG; ++j) o[j] *= corr;
    const int nk = pos - kb + 1 < 32 ? pos - kb + 1 : 32;
    for (int j = 0; j < nk; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const size_t bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
      if (pj == 0.f) continue;
      const T* vp = cache + bj;
#pragma unroll
      for (int r = 0; r < NREG; ++r) {
        const int i = lane + 32 * r;
        if (i < rank) o[r] = fmaf(pj, to_f(vp[i]), o[r]);
      }
    }
    m = m_new;
  }
  // the weighted latent, then the head's value matrix and the gate
  __syncwarp();
  const float inv = 1.0f / l;
#pragma unroll
  for (int r = 0; r < NREG; ++r) {
    const int i = lane + 32 * r;
    if (i < rank) qs[i] = o[r] * inv;
  }
  __syncwarp();
  T* orow = out + (size_t)t * ld_out + (size_t)h * dv;
  const T* grow = gate ? gate + (size_t)t * ld_gate + (size_t)h * dv : nullptr;
  for (int j = 0; j < dv; ++j) {
    const TW* wr = wuv + ((size_t)h * dv + j) * rank;
    float acc = 0.f;
    for (int r = lane; r < rank; r += 32) acc = fmaf(to_f(wr[r]), qs[r], acc);
    acc = warp_sum(acc);
    if (lane == 0) {
      if (grow) acc *= 1.0f / (1.0f + expf(-to_f(grow[j])));
      orow[j] = from_f<T>(acc);
    }
  }
}

extern "C" int qv_latent_attention_generic(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                                           const void* cache, const void* wuk, const void* wuv, const int* tok_pos,
                                           const int* tok_seg, const int* block_table, int max_blocks, int T, int H, int dn,
                                           int dr, int dv, int rank, int page, int window, float scale, int dt, int w_dt,
                                           void* stream) {
  if (T <= 0) return 0;
  if (rank > LAT_MAX_RANK || rank <= 0 || dn < 0 || dr < 0 || dv <= 0) return QV_ERR_UNSUPPORTED;
  const size_t smem = (size_t)4 * (rank + dr + dn) * sizeof(float);
  if (smem > 200 * 1024) return QV_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  int done = 0;
  while (done < T) {                               // rows are independent; the grid's second dimension is limited
    const int n = T - done < 65535 ? T - done : 65535;
    const size_t esz = dt == QV_DT_F32 ? 4 : 2;
    void* o = (char*)out + (size_t)done * ld_out * esz;
    const void* qq = (const char*)q + (size_t)done * ld_q * esz;
    const void* gg = gate ? (const char*)gate + (size_t)done * ld_gate * esz : nullptr;
    dim3 grid((H + 3) / 4, n);
    int rc;
#define LAT_GENERIC(TT, TW)                                                                                              \
  do {                                                                                                                   \
    if (smem > 48 * 1024)                                                                                                \
      cudaFuncSetAttribute(latent_attention_generic_kernel<TT, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    rc = qv_launch(latent_attention_generic_kernel<TT, TW>, grid, dim3(128), smem, st, (TT*)o, ld_out, (const TT*)qq, ld_q, \
                   (const TT*)gg, ld_gate, (const TT*)cache, (const TW*)wuk, (const TW*)wuv, tok_pos + done, tok_seg + done, \
                   block_table, max_blocks, H, dn, dr, dv, rank, page, window, scale);                                   \
  } while (0)
    if (dt == QV_DT_F32 && w_dt == QV_DT_F32) LAT_GENERIC(float, float);
    else if (dt == QV_DT_BF16 && w_dt == QV_DT_BF16) LAT_GENERIC(bf16, bf16);
    else if (dt == QV_DT_BF16 && w_dt == QV_DT_F32) LAT_GENERIC(bf16, float);
    else if (dt == QV_DT_F32 && w_dt == QV_DT_BF16) LAT_GENERIC(float, bf16);
    else return QV_ERR_UNSUPPORTED;
#undef LAT_GENERIC
    if (rc) return rc;
    done += n;
  }
  return 0;
}
