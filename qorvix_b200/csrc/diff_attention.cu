// Differential attention over a paged cache of rows: every head has two query/key maps over one set of values,
//   a_m = softmax_j((q_m . k_m,j) * scale) V      for the two maps m = 1, 2 (causal, optionally the last `window` keys),
//   o = a_1 - lam * a_2;   out = o / sqrt(mean(o^2) + eps) * post            (mean over the head's value entries).
//
// qv_diff_prepare            per token: bias added to the projection's sums, every map of q and k divided by its root
//                            mean square and weighted, the first `rot` entries of each map rotated (pairs i, i + rot/2,
//                            cos/sin from a table row of the token's position); q goes to a dense buffer, k and v (with
//                            its bias) to the token's cache row [k: G x 2n | v: G x dv].  All arithmetic float32.
// qv_diff_attention_generic  one warp per (token, head), float32 arithmetic whatever the storage type, any sizes; keys in
//                            blocks of 32 aligned to absolute positions with running maxima and sums for both maps, so a
//                            position's result depends on the position and the cache contents only.
#include "common.cuh"

#define DIFF_MAX_DV 512

template <typename TP, typename T>
__global__ void __launch_bounds__(256) diff_prepare_kernel(T* __restrict__ q_out, int ld_q, const TP* __restrict__ proj, int ld_p,
                                                           const float* __restrict__ bias, const float* __restrict__ qw,
                                                           const float* __restrict__ kw, float eps, const float2* __restrict__ cos_sin,
                                                           int table_rows, const int* __restrict__ tok_pos, const int* __restrict__ tok_seg,
                                                           const int* __restrict__ block_table, int max_blocks, T* __restrict__ cache,
                                                           int H, int G, int n, int dv, int rot, int page) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, lane = threadIdx.x & 31;
  const int unit = blockIdx.y * 8 + (threadIdx.x >> 5);      // 2H maps of q, 2G maps of k, G heads of v
  const int nq = 2 * H, nk = 2 * G;
  if (unit >= nq + nk + G) return;
  const int pos = tok_pos[t];
  const size_t width = (size_t)G * (2 * n + dv);
  T* crow = nullptr;
  if (cache) {
    const int pg = block_table[(size_t)tok_seg[t] * max_blocks + pos / page];
    crow = cache + ((size_t)pg * page + pos % page) * width;
  }
  const TP* prow = proj + (size_t)t * ld_p;
  if (unit < nq + nk) {
    const bool is_q = unit < nq;
    if (!is_q && !crow) return;
    const int col0 = unit * n;                               // the k maps follow the q maps in the projection's columns
    const TP* src = prow + col0;
    const float* b = bias ? bias + col0 : nullptr;
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) {
      const float x = to_f(src[i]) + (b ? b[i] : 0.f);
      ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    const float* w = is_q ? qw : kw;
    T* dst = is_q ? q_out + (size_t)t * ld_q + col0 : crow + (size_t)(unit - nq) * n;
    const int half = rot >> 1;
    const float2* cs = cos_sin ? cos_sin + (size_t)(pos < table_rows ? pos : table_rows - 1) * half : nullptr;
    for (int i = lane; i < half; i += 32) {
      const float u = (to_f(src[i]) + (b ? b[i] : 0.f)) * inv * w[i];
      const float v = (to_f(src[i + half]) + (b ? b[i + half] : 0.f)) * inv * w[i + half];
      const float2 c = cs[i];
      dst[i] = from_f<T>(u * c.x - v * c.y);
      dst[i + half] = from_f<T>(v * c.x + u * c.y);
    }
    for (int i = rot + lane; i < n; i += 32) dst[i] = from_f<T>((to_f(src[i]) + (b ? b[i] : 0.f)) * inv * w[i]);
  } else if (crow) {
    const int vh = unit - nq - nk;
    const int col0 = (nq + nk) * n + vh * dv;
    const TP* src = prow + col0;
    T* dst = crow + (size_t)G * 2 * n + (size_t)vh * dv;
    for (int i = lane; i < dv; i += 32) dst[i] = from_f<T>(to_f(src[i]) + (bias ? bias[col0 + i] : 0.f));
  }
}

extern "C" int qv_diff_prepare(void* q_out, int ld_q, const void* proj, int ld_p, const float* bias, const float* qw, const float* kw,
                               float eps, const float* cos_sin, int table_rows, const int* tok_pos, const int* tok_seg,
                               const int* block_table, int max_blocks, void* cache, int T, int H, int G, int n, int dv, int rot, int page,
                               int proj_dt, int dt, void* stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > n || (rot & 1) || (rot > 0 && !cos_sin) || H <= 0 || G <= 0) return QV_ERR_UNSUPPORTED;
  const int units = 2 * H + 3 * G;
  if ((units + 7) / 8 > 65535) return QV_ERR_TOO_LARGE;
  const dim3 grid(T, (units + 7) / 8);
  cudaStream_t st = (cudaStream_t)stream;
#define PREP(TP, TT)                                                                                                              \
  return qv_launch(diff_prepare_kernel<TP, TT>, grid, dim3(256), 0, st, (TT*)q_out, ld_q, (const TP*)proj, ld_p, bias, qw, kw, eps, \
                   (const float2*)cos_sin, table_rows, tok_pos, tok_seg, block_table, max_blocks, (TT*)cache, H, G, n, dv, rot, page)
  if (proj_dt == QV_DT_F32 && dt == QV_DT_F32) PREP(float, float);
  if (proj_dt == QV_DT_F32 && dt == QV_DT_BF16) PREP(float, bf16);
  if (proj_dt == QV_DT_BF16 && dt == QV_DT_BF16) PREP(bf16, bf16);
#undef PREP
  return QV_ERR_UNSUPPORTED;
}

template <typename T>
__global__ void __launch_bounds__(128) diff_attention_generic_kernel(
    T* __restrict__ out, int ld_out, const T* __restrict__ q, int ld_q, const T* __restrict__ cache, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_seg, const int* __restrict__ block_table, int max_blocks, int H, int G, int n, int dv, int page,
    int window, float scale, float lam, float eps, float post) {
  extern __shared__ float qs_all[];              // 4 warps x 2n floats
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x * 4 + warp;
  const int t = blockIdx.y;
  if (h >= H) return;                            // whole warp leaves together
  float* qs = qs_all + (size_t)warp * 2 * n;
  const T* qrow = q + (size_t)t * ld_q + (size_t)h * 2 * n;
  for (int i = lane; i < 2 * n; i += 32) qs[i] = to_f(qrow[i]);
  __syncwarp();
  const int pos = tok_pos[t];
  const int* bt = block_table + (size_t)tok_seg[t] * max_blocks;
  const int g = h / (H / G);
  const int lo = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
  const size_t width = (size_t)G * (2 * n + dv);
  const size_t k_off = (size_t)g * 2 * n, v_off = (size_t)G * 2 * n + (size_t)g * dv;

  constexpr int NREG = DIFF_MAX_DV / 32;
  float o1[NREG], o2[NREG];
#pragma unroll
  for (int j = 0; j < NREG; ++j) o1[j] = o2[j] = 0.f;
  float m1 = -INFINITY, l1 = 0.f, m2 = -INFINITY, l2 = 0.f;
  for (int kb = (lo >> 5) << 5; kb <= pos; kb += 32) {
    const int tk = kb + lane;
    const bool valid = tk >= lo && tk <= pos;
    size_t base = 0;
    float s1 = -INFINITY, s2 = -INFINITY;
    if (valid) {
      base = ((size_t)bt[tk / page] * page + (size_t)(tk % page)) * width;
      const T* kp = cache + base + k_off;
      float d1 = 0.f, d2 = 0.f;
      for (int i = 0; i < n; ++i) d1 = fmaf(qs[i], to_f(kp[i]), d1);
      for (int i = 0; i < n; ++i) d2 = fmaf(qs[n + i], to_f(kp[n + i]), d2);
      s1 = d1 * scale;
      s2 = d2 * scale;
    }
    const float m1n = fmaxf(m1, warp_max(s1)), m2n = fmaxf(m2, warp_max(s2));    // finite: the block holds a valid key
    const float p1 = valid ? expf(s1 - m1n) : 0.f, p2 = valid ? expf(s2 - m2n) : 0.f;
    const float c1 = expf(m1 - m1n), c2 = expf(m2 - m2n);
    l1 = l1 * c1 + warp_sum(p1);
    l2 = l2 * c2 + warp_sum(p2);
#pragma unroll
    for (int j = 0; j < NREG; ++j) { o1[j] *= c1; o2[j] *= c2; }
    const int nkeys = pos - kb + 1 < 32 ? pos - kb + 1 : 32;
    for (int j = 0; j < nkeys; ++j) {
      const float p1j = __shfl_sync(0xffffffffu, p1, j), p2j = __shfl_sync(0xffffffffu, p2, j);
      const size_t bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
      if (p1j == 0.f && p2j == 0.f) continue;    // before the window, or underflowed in both maps
      const T* vp = cache + bj + v_off;
#pragma unroll
      for (int r = 0; r < NREG; ++r) {
        const int i = lane + 32 * r;
        if (i < dv) {
          const float v = to_f(vp[i]);
          o1[r] = fmaf(p1j, v, o1[r]);
          o2[r] = fmaf(p2j, v, o2[r]);
        }
      }
    }
    m1 = m1n;
    m2 = m2n;
  }
  const float i1 = 1.0f / l1, i2 = 1.0f / l2;
  float ss = 0.f;
#pragma unroll
  for (int r = 0; r < NREG; ++r) {
    const int i = lane + 32 * r;
    o1[r] = i < dv ? o1[r] * i1 - lam * (o2[r] * i2) : 0.f;
    ss = fmaf(o1[r], o1[r], ss);
  }
  ss = warp_sum(ss);
  const float inv = post / sqrtf(ss / (float)dv + eps);
  T* orow = out + (size_t)t * ld_out + (size_t)h * dv;
#pragma unroll
  for (int r = 0; r < NREG; ++r) {
    const int i = lane + 32 * r;
    if (i < dv) orow[i] = from_f<T>(o1[r] * inv);
  }
}

extern "C" int qv_diff_attention_generic(void* out, int ld_out, const void* q, int ld_q, const void* cache, const int* tok_pos,
                                         const int* tok_seg, const int* block_table, int max_blocks, int T, int H, int G, int n, int dv,
                                         int page, int window, float scale, float lam, float eps, float post, int dt, void* stream) {
  if (T <= 0) return 0;
  if (dv > DIFF_MAX_DV || dv <= 0 || n <= 0 || G <= 0 || H % G) return QV_ERR_UNSUPPORTED;
  const size_t smem = (size_t)4 * 2 * n * sizeof(float);
  if (smem > 48 * 1024) return QV_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t esz = dt == QV_DT_F32 ? 4 : 2;
  for (int done = 0; done < T; done += 65535) {            // rows are independent: several launches for very many tokens
    const int rows = T - done < 65535 ? T - done : 65535;
    const dim3 grid((H + 3) / 4, rows);
    int rc = QV_ERR_UNSUPPORTED;
    QV_DISPATCH_DT(dt, TT,
                   rc = qv_launch(diff_attention_generic_kernel<TT>, grid, dim3(128), smem, st, (TT*)((char*)out + (size_t)done * ld_out * esz),
                                  ld_out, (const TT*)((const char*)q + (size_t)done * ld_q * esz), ld_q, (const TT*)cache, tok_pos + done,
                                  tok_seg + done, block_table, max_blocks, H, G, n, dv, page, window, scale, lam, eps, post));
    if (rc) return rc;
  }
  return 0;
}
