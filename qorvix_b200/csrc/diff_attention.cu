// Differential attention over a paged cache of rows: every head has two query/key maps over one set of values,
//   a_m = softmax_j((q_m . k_m,j) * scale) V      for the two maps m = 1, 2 (causal, optionally the last `window` keys),
//   o = a_1 - lam * a_2;   out = o / sqrt(mean(o^2) + eps) * post            (mean over the head's value entries).
//
// qv_diff_prepare            per token (a CTA): bias added to the projection's sums, every map of q and k divided by its
//                            root mean square and weighted, the first `rot` entries of each map rotated (pairs i, i + rot/2,
//                            cos/sin from a table row of the token's position); q goes to a dense buffer, k and v (with
//                            its bias) to the token's cache row [k: G x 2n | v: G x dv].  All arithmetic float32.
// qv_diff_attention_generic  one warp per (token, head), float32 arithmetic whatever the storage type, any sizes; keys in
//                            blocks of 32 aligned to absolute positions with running maxima and sums for both maps, so a
//                            position's result depends on the position and the cache contents only.
#include "common.cuh"

#define DIFF_MAX_DV 512

// A CTA serves a token (or, in steps of few tokens, a share of a token's maps): the token's row of the projection (plus bias)
// is brought into shared memory by all threads at once, then every warp takes maps of q and k (norm, weight, rotation) and
// heads of v in turn and writes them out.
template <typename TP, typename T>
__global__ void __launch_bounds__(256) diff_prepare_kernel(T* __restrict__ q_out, int ld_q, const TP* __restrict__ proj, int ld_p,
                                                           const float* __restrict__ bias, const float* __restrict__ qw,
                                                           const float* __restrict__ kw, float eps, const float2* __restrict__ cos_sin,
                                                           int table_rows, const int* __restrict__ tok_pos, const int* __restrict__ tok_seg,
                                                           const int* __restrict__ block_table, int max_blocks, T* __restrict__ cache,
                                                           int H, int G, int n, int dv, int rot, int page) {
  extern __shared__ float prep_row[];                        // the token's (H + G) * 2n + G * dv sums, bias added
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nq = 2 * H, nk = 2 * G;
  const int cols = (nq + nk) * n + G * dv;
  const TP* prow = proj + (size_t)t * ld_p;
  if (sizeof(TP) == 4 && (cols & 3) == 0 && (ld_p & 3) == 0 && (((uintptr_t)proj | (uintptr_t)bias) & 15) == 0) {
    for (int i = threadIdx.x * 4; i < cols; i += 256 * 4) {
      float4 v = *(const float4*)((const float*)prow + i);
      if (bias) {
        const float4 bv = *(const float4*)(bias + i);
        v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
      }
      *(float4*)(prep_row + i) = v;
    }
  } else {
    for (int i = threadIdx.x; i < cols; i += 256) prep_row[i] = to_f(prow[i]) + (bias ? bias[i] : 0.f);
  }
  const int pos = tok_pos[t];
  const size_t width = (size_t)G * (2 * n + dv);
  T* crow = nullptr;
  if (cache) {
    const int pg = block_table[(size_t)tok_seg[t] * max_blocks + pos / page];
    crow = cache + ((size_t)pg * page + pos % page) * width;
  }
  const int half = rot >> 1;
  const float2* cs = cos_sin ? cos_sin + (size_t)(pos < table_rows ? pos : table_rows - 1) * half : nullptr;
  __syncthreads();
  for (int unit = blockIdx.y * 8 + warp; unit < nq + nk + G; unit += 8 * gridDim.y) {     // 2H maps of q, 2G maps of k, G heads of v
    if (unit < nq + nk) {
      const bool is_q = unit < nq;
      if (!is_q && !crow) continue;
      const int col0 = unit * n;                             // the k maps follow the q maps in the projection's columns
      const float* src = prep_row + col0;
      float ss = 0.f;
      for (int i = lane; i < n; i += 32) ss = fmaf(src[i], src[i], ss);
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)n + eps);
      const float* w = is_q ? qw : kw;
      T* dst = is_q ? q_out + (size_t)t * ld_q + col0 : crow + (size_t)(unit - nq) * n;
      for (int i = lane; i < half; i += 32) {
        const float u = src[i] * inv * w[i];
        const float v = src[i + half] * inv * w[i + half];
        const float2 c = cs[i];
        dst[i] = from_f<T>(u * c.x - v * c.y);
        dst[i + half] = from_f<T>(v * c.x + u * c.y);
      }
      for (int i = rot + lane; i < n; i += 32) dst[i] = from_f<T>(src[i] * inv * w[i]);
    } else if (crow) {
      const int vh = unit - nq - nk;
      const float* src = prep_row + (nq + nk) * n + vh * dv;
      T* dst = crow + (size_t)G * 2 * n + (size_t)vh * dv;
      for (int i = lane; i < dv; i += 32) dst[i] = from_f<T>(src[i]);
    }
  }
}

extern "C" int qv_diff_prepare(void* q_out, int ld_q, const void* proj, int ld_p, const float* bias, const float* qw, const float* kw,
                               float eps, const float* cos_sin, int table_rows, const int* tok_pos, const int* tok_seg,
                               const int* block_table, int max_blocks, void* cache, int T, int H, int G, int n, int dv, int rot, int page,
                               int proj_dt, int dt, void* stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > n || (rot & 1) || (rot > 0 && !cos_sin) || H <= 0 || G <= 0) return QV_ERR_UNSUPPORTED;
  const size_t smem = (size_t)((H + G) * 2 * n + G * dv) * sizeof(float);
  if (smem > 200 * 1024) return QV_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  // few tokens: a token's maps are spread over several CTAs (each brings the row in for itself), so that the step fills more SMs
  const int units = 2 * H + 3 * G;
  const int spread = T <= 32 ? ((units + 7) / 8 < 65535 ? (units + 7) / 8 : 65535) : 1;
#define PREP(TP, TT)                                                                                                              \
  do {                                                                                                                            \
    if (smem > 48 * 1024) cudaFuncSetAttribute(diff_prepare_kernel<TP, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    return qv_launch(diff_prepare_kernel<TP, TT>, dim3(T, spread), dim3(256), smem, st, (TT*)q_out, ld_q, (const TP*)proj, ld_p, bias, qw, kw, \
                     eps, (const float2*)cos_sin, table_rows, tok_pos, tok_seg, block_table, max_blocks, (TT*)cache, H, G, n, dv, rot, \
                     page);                                                                                                       \
  } while (0)
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

// ---------------------------------------------------------------- tensor cores (bfloat16)
// qv_diff_attention_tc       a CTA serves a tile of 16 * MW query rows of one segment and one head with 2 * MW warps: warps
//                            0..MW-1 run map 1 and warps MW..2MW-1 map 2, each over 16 rows; blocks of 32 keys (both maps' key
//                            entries and the values) come through a cp.async ring of four stages that both maps read; Q.K^T and P.V as
//                            mma.sync m16n8k16 with float32 sums, softmax in float32 (base 2), every weight entering P.V as three
//                            bfloat16 terms that together hold its 24 bits; at the end map 2's warps leave
//                            their normalised rows in shared memory and map 1's warps form a1 - lam * a2, the root mean square
//                            over the head's values and the output.  Map and value sizes are padded with zeros up to the
//                            template's (NT, DVT), so one instantiation serves all sizes below it (multiples of 8).
//                            Single query tokens take a tile whose rows are the query heads of one key/value head (the keys are
//                            read once for the group); their keys may be cut into slices (grid.x = slices): the two maps'
//                            running maxima, sums and unnormalised rows then go to a workspace that the merge kernel finishes.
#define DIFF_KB 32

__device__ __forceinline__ void dcp_async16(void* smem, const void* gmem, int bytes) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void dldsm4(uint32_t* r, const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void dldsm4t(uint32_t* r, const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void dmma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t dpack(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&h;
}

template <int NT, int DVT, int MW, bool GROUPED, int STAGES, int DIFF_P_TERMS>
__global__ void __launch_bounds__(MW == 1 ? 128 : 64 * MW, MW == 1 ? 1 : (DVT <= 128 ? 2 : 1)) diff_attention_tc_kernel(
    bf16* __restrict__ out, int ld_out, const bf16* __restrict__ q, int ld_q, const bf16* __restrict__ cache,
    const int* __restrict__ seg_q_start, const int* __restrict__ seg_pos0, const int* __restrict__ block_table, int max_blocks,
    int H, int G, int n, int dv, int page, int page_shift, int window, float scale_log2, float lam, float eps, float post,
    float* __restrict__ partial, int splits) {
  // GROUPED (single query tokens, MW == 1): the tile's rows are the query heads of one key/value head, which all see the
  // same keys, so those are read once for the group.  Else the rows are tokens of one segment and one head.  With MW == 1
  // two more warps only help to copy.
  constexpr int TM = 16 * MW, THREADS = MW == 1 ? 128 : 64 * MW, NWARPS = THREADS / 32;
  constexpr int LDK = 2 * NT + 8, LDV = DVT + 8;          // padded rows: ldmatrix without bank conflicts
  constexpr int STAGE = DIFF_KB * (LDK + LDV);            // elements of one stage (keys of both maps, then values)
  extern __shared__ __align__(16) unsigned char diff_smem[];
  bf16* Qs = (bf16*)diff_smem;                            // [TM][LDK]
  bf16* ring = Qs + TM * LDK;                             // [STAGES][STAGE]
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool computes = warp < 2 * MW;
  const int mp = computes ? warp / MW : 0, r0 = (warp % MW) * 16;        // this warp's map and first row of the tile
  const int seg = blockIdx.y;
  const int hpg = H / G;
  // grouped: grid (slices, tokens, key/value heads); else (heads, segments, tiles) with the last tiles of the segments,
  // which see the most keys, first in the order CTAs are handed out, so that the short ones fill the SMs at the end
  const int g = GROUPED ? blockIdx.z : blockIdx.x / hpg;
  const int h = GROUPED ? g * hpg : blockIdx.x;           // the (first) head of the tile
  const int q0 = seg_q_start[seg], len = seg_q_start[seg + 1] - q0;
  const int row0 = GROUPED ? 0 : (gridDim.z - 1 - blockIdx.z) * TM;
  if (!GROUPED && row0 >= len) return;
  const int rows = GROUPED ? hpg : (len - row0 < TM ? len - row0 : TM);
  const int pos0 = seg_pos0[seg] + row0;                  // position of the tile's first row
  const size_t width = (size_t)G * (2 * n + dv);
  const int* bt = block_table + (size_t)seg * max_blocks;
  const int kmin = window > 0 ? (pos0 - window + 1 > 0 ? pos0 - window + 1 : 0) : 0;
  const int kmax = GROUPED ? pos0 : pos0 + rows - 1;
  int kb0 = (kmin / DIFF_KB) * DIFF_KB;
  int nb = (kmax - kb0) / DIFF_KB + 1;
  if (GROUPED && splits > 1) {                            // this slice's share of the blocks
    const int per = (nb + splits - 1) / splits;
    const int b_lo = blockIdx.x * per, b_hi = b_lo + per < nb ? b_lo + per : nb;
    kb0 += b_lo * DIFF_KB;
    nb = b_hi - b_lo;                                     // may be <= 0: an empty slice leaves an empty partial
  }

  // A warp copies whole key rows, every lane its own 16-byte pieces of the row: where a lane's pieces lie in the row and
  // in a stage is worked out once; per key only the row's address is left to find.
  constexpr int KC = 2 * NT / 8, VC = DVT / 8;            // 16-byte pieces of a key row (both maps) and of a value row
  constexpr int NP = (KC + VC + 31) / 32;                 // pieces a lane copies per key
  int piece_src[NP], piece_dst[NP], piece_ld[NP];         // element offset in the cache row (-1: zeros), in the stage, stage row length
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int cc = lane + 32 * i;
    piece_src[i] = -1;
    piece_dst[i] = 0;
    piece_ld[i] = 0;
    if (cc < KC) {
      const int m = (cc * 8) / NT, within = cc * 8 - m * NT;
      if (within < n) piece_src[i] = g * 2 * n + m * n + within;
      piece_dst[i] = cc * 8;
      piece_ld[i] = LDK;
    } else if (cc < KC + VC) {
      const int col = (cc - KC) * 8;
      if (col < dv) piece_src[i] = G * 2 * n + g * dv + col;
      piece_dst[i] = DIFF_KB * LDK + col;
      piece_ld[i] = LDV;
    }
  }
  auto load_block = [&](int stage, int kb) {
    bf16* base = ring + stage * STAGE;
    // the block's page numbers in one load (lane l: key kb + l), handed out by shuffles: a look-up per key would
    // put a round trip to memory ahead of every row's copies
    static_assert(DIFF_KB == 32, "one lane a key");
    int page_of_lane = 0;
    {
      const int key = kb + lane;
      if (key >= kmin && key <= kmax) page_of_lane = bt[page_shift >= 0 ? key >> page_shift : key / page];
    }
    for (int j = warp; j < DIFF_KB; j += NWARPS) {
      const int key = kb + j;
      const bool kin = key >= kmin && key <= kmax;
      const int page_id = __shfl_sync(0xffffffffu, page_of_lane, j);
      const int in_page = page_shift >= 0 ? key & (page - 1) : key % page;
      const bf16* row = cache + ((size_t)page_id * page + (size_t)in_page) * width;       // a key outside the range reads nothing
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        if (NP * 32 == KC + VC || lane + 32 * i < KC + VC) {
          const bool ok = kin && piece_src[i] >= 0;
          dcp_async16(base + j * piece_ld[i] + piece_dst[i], ok ? row + piece_src[i] : cache, ok ? 16 : 0);
        }
      }
    }
  };
  {   // the tile's queries, both maps, zero-padded
    for (int r = warp; r < TM; r += NWARPS) {
      const bf16* qrow = GROUPED ? q + (size_t)q0 * ld_q + (size_t)(h + r) * 2 * n : q + (size_t)(q0 + row0 + r) * ld_q + (size_t)h * 2 * n;
#pragma unroll
      for (int cc = lane; cc < KC; cc += 32) {
        const int m = (cc * 8) / NT, within = cc * 8 - m * NT;
        const bool ok = r < rows && within < n;
        dcp_async16(Qs + r * LDK + cc * 8, ok ? qrow + m * n + within : q, ok ? 16 : 0);
      }
    }
  }
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {               // one group a stage, empty past the end, so that the counts below hold
    if (st < nb) load_block(st, kb0 + st * DIFF_KB);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  const int gr = lane >> 2, tg = lane & 3;                // fragment row (and row + 8), column pair
  int lo[2], hi[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = r0 + gr + 8 * e;
    const int p = GROUPED ? pos0 : pos0 + r;
    hi[e] = r < rows ? p : -1;
    lo[e] = window > 0 ? (p - window + 1 > 0 ? p - window + 1 : 0) : 0;
  }
  // keys any row of this warp can see, and keys all of its rows see
  const int p_first = GROUPED ? pos0 : pos0 + r0, p_last = GROUPED ? pos0 : pos0 + (r0 + 15 < rows - 1 ? r0 + 15 : rows - 1);
  const int w_lo = window > 0 ? (p_first - window + 1 > 0 ? p_first - window + 1 : 0) : 0;
  const int w_hi = r0 < rows ? p_last : -1;
  const int all_lo = window > 0 ? (p_last - window + 1 > 0 ? p_last - window + 1 : 0) : 0;
  const int all_hi = (r0 + 15 < rows) ? p_first : -1;     // a tile with rows past its end masks them in every block
  float o[DVT / 8][4];
#pragma unroll
  for (int i = 0; i < DVT / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

  for (int b = 0; b < nb; ++b) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();                         // block b has landed for everyone; the stage filled next was read a round ago
    if (b + STAGES - 1 < nb) load_block((b + STAGES - 1) % STAGES, kb0 + (b + STAGES - 1) * DIFF_KB);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const int kb = kb0 + b * DIFF_KB;
    if (computes && kb <= w_hi && kb + DIFF_KB - 1 >= w_lo) {
      const bf16* Ks = ring + (b % STAGES) * STAGE;
      const bf16* Vs = Ks + DIFF_KB * LDK;
      float s[DIFF_KB / 8][4];
#pragma unroll
      for (int i = 0; i < DIFF_KB / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kc = 0; kc < NT / 16; ++kc) {
        uint32_t qf[4];                      // the queries' fragments come from shared memory block by block: registers are what limits the CTAs an SM holds
        dldsm4(qf, Qs + (r0 + (lane & 15)) * LDK + mp * NT + kc * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int pr = 0; pr < DIFF_KB / 16; ++pr) {
          uint32_t bfr[4];
          dldsm4(bfr, Ks + (pr * 16 + (lane >> 4) * 8 + (lane & 7)) * LDK + mp * NT + kc * 16 + ((lane >> 3) & 1) * 8);
          dmma(s[2 * pr], qf, bfr[0], bfr[1]);
          dmma(s[2 * pr + 1], qf, bfr[2], bfr[3]);
        }
      }
      float mx[2] = {-INFINITY, -INFINITY};
      if (kb >= all_lo && kb + DIFF_KB - 1 <= all_hi) {   // every row of the warp sees the whole block: nothing to mask
#pragma unroll
        for (int i = 0; i < DIFF_KB / 8; ++i) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[i][e] *= scale_log2;
            mx[e >> 1] = fmaxf(mx[e >> 1], s[i][e]);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < DIFF_KB / 8; ++i) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = kb + i * 8 + 2 * tg + (e & 1), r = e >> 1;
            const float v = (key >= lo[r] && key <= hi[r]) ? s[i][e] * scale_log2 : -INFINITY;
            s[i][e] = v;
            mx[r] = fmaxf(mx[r], v);
          }
        }
      }
      float corr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(mrow[r], mx[r]);
        corr[r] = (m_new == -INFINITY) ? 1.f : exp2f(mrow[r] - m_new);     // a row that has seen no key keeps -inf
        mrow[r] = m_new;
        lrow[r] *= corr[r];
      }
      const float mref[2] = {mrow[0] == -INFINITY ? 0.f : mrow[0], mrow[1] == -INFINITY ? 0.f : mrow[1]};
#pragma unroll
      for (int i = 0; i < DIFF_KB / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const float p = exp2f(s[i][e] - mref[r]);       // a masked score is -inf: its weight is 0
          s[i][e] = p;
          lrow[r] += p;
        }
      }
      if (!__all_sync(0xffffffffu, corr[0] == 1.f && corr[1] == 1.f)) {      // no row's maximum moved: nothing to scale down
#pragma unroll
        for (int i = 0; i < DVT / 8; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
      }
      // The weights stay 32-bit in the product with the values: each is the sum of DIFF_P_TERMS bfloat16 terms (the value
      // rounded, then what is left, rounded again, ...; three terms hold all 24 bits), and every term is multiplied.
#pragma unroll
      for (int kc = 0; kc < DIFF_KB / 16; ++kc) {
        float w[8] = {s[2 * kc][0], s[2 * kc][1], s[2 * kc][2], s[2 * kc][3], s[2 * kc + 1][0], s[2 * kc + 1][1], s[2 * kc + 1][2], s[2 * kc + 1][3]};
        uint32_t a[DIFF_P_TERMS][4];
#pragma unroll
        for (int term = 0; term < DIFF_P_TERMS; ++term) {
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const __nv_bfloat162 pr = __floats2bfloat162_rn(w[2 * x], w[2 * x + 1]);
            a[term][x] = *(const uint32_t*)&pr;
            if (term + 1 < DIFF_P_TERMS) {
              w[2 * x] -= __low2float(pr);
              w[2 * x + 1] -= __high2float(pr);
            }
          }
        }
#pragma unroll
        for (int nt = 0; nt < DVT / 16; ++nt) {
          uint32_t bfr[4];
          dldsm4t(bfr, Vs + (kc * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + nt * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int term = DIFF_P_TERMS - 1; term >= 0; --term) {      // the small terms first
            dmma(o[2 * nt], a[term], bfr[0], bfr[1]);
            dmma(o[2 * nt + 1], a[term], bfr[2], bfr[3]);
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                           // all warps are past their last block: the ring is free
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
  }
  if (GROUPED && splits > 1) {
    // [token][head][slice][map][m, l, DVT values]; the tile's rows are the group's heads
    if (computes) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int row = gr + 8 * e;
        if (row >= rows) continue;
        float* dst = partial + ((((size_t)seg * H + h + row) * splits + blockIdx.x) * 2 + mp) * (DVT + 2);
        if (tg == 0) { dst[0] = mrow[e]; dst[1] = lrow[e]; }
#pragma unroll
        for (int i = 0; i < DVT / 8; ++i) { dst[2 + i * 8 + 2 * tg] = o[i][2 * e]; dst[2 + i * 8 + 2 * tg + 1] = o[i][2 * e + 1]; }
      }
    }
    return;
  }
  const float inv_l[2] = {lrow[0] > 0.f ? 1.0f / lrow[0] : 0.f, lrow[1] > 0.f ? 1.0f / lrow[1] : 0.f};
  float* a2 = (float*)ring;                  // [TM][DVT + 1] float32, over the ring (all warps are past their last block)
  constexpr int LDA = DVT + 1;
  if (computes && mp == 1) {
#pragma unroll
    for (int i = 0; i < DVT / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) a2[(r0 + gr + 8 * (e >> 1)) * LDA + i * 8 + 2 * tg + (e & 1)] = o[i][e] * inv_l[e >> 1];
    }
  }
  __syncthreads();
  if (computes && mp == 0) {
    float ss[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < DVT / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float v = o[i][e] * inv_l[e >> 1] - lam * a2[(r0 + gr + 8 * (e >> 1)) * LDA + i * 8 + 2 * tg + (e & 1)];
        o[i][e] = v;                         // columns from dv on are zero in both maps (their values were filled with zeros)
        ss[e >> 1] = fmaf(v, v, ss[e >> 1]);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], 1);
      ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], 2);
      ss[r] = post / sqrtf(ss[r] / (float)dv + eps);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = r0 + gr + 8 * r;
      if (row >= rows) continue;
      bf16* orow = GROUPED ? out + (size_t)q0 * ld_out + (size_t)(h + row) * dv : out + (size_t)(q0 + row0 + row) * ld_out + (size_t)h * dv;
#pragma unroll
      for (int i = 0; i < DVT / 8; ++i) {
        const int col = i * 8 + 2 * tg;
        if (col < dv) *(__nv_bfloat162*)(orow + col) = __floats2bfloat162_rn(o[i][2 * r] * ss[r], o[i][2 * r + 1] * ss[r]);
      }
    }
  }
}

// Finishes single tokens whose keys were cut into slices: per (token, head) the slices' maxima, sums and rows of both maps
// are merged, then o = a1 - lam * a2, the root mean square over dv, the output.  One warp each; lane s holds slice s's
// maximum and sum (at most 32 slices), and the rows are fetched four slices at a time so that their loads overlap.
template <int DVT>
__global__ void __launch_bounds__(128) diff_merge_kernel(bf16* __restrict__ out, int ld_out, const float* __restrict__ partial, int T, int H,
                                                         int dv, int splits, float lam, float eps, float post) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int idx = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (idx >= T * H) return;
  const int t = idx / H, h = idx - t * H;
  constexpr int NR = DVT / 32;
  constexpr size_t STRIDE = 2 * (DVT + 2);                 // floats from a slice to the next (both maps)
  const float* base = partial + (size_t)idx * splits * STRIDE;
  float wgt[2], a[2][NR];
#pragma unroll
  for (int mp = 0; mp < 2; ++mp) {
    const float* p = base + (size_t)lane * STRIDE + mp * (DVT + 2);
    const float ms = lane < splits ? p[0] : -INFINITY, ls = lane < splits ? p[1] : 0.f;
    const float m = warp_max(ms);
    wgt[mp] = ms == -INFINITY ? 0.f : exp2f(ms - m);
    const float l = warp_sum(wgt[mp] * ls);               // a fixed order: the result does not depend on the batch
    wgt[mp] *= l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r) a[mp][r] = 0.f;
  }
  for (int s0 = 0; s0 < splits; s0 += 4) {
    float v[4][2][NR];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
#pragma unroll
      for (int mp = 0; mp < 2; ++mp) {
#pragma unroll
        for (int r = 0; r < NR; ++r) v[u][mp][r] = s0 + u < splits ? base[(size_t)(s0 + u) * STRIDE + mp * (DVT + 2) + 2 + lane + 32 * r] : 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
#pragma unroll
      for (int mp = 0; mp < 2; ++mp) {
        const float w = __shfl_sync(0xffffffffu, wgt[mp], (s0 + u) & 31);
#pragma unroll
        for (int r = 0; r < NR; ++r) a[mp][r] = fmaf(w, v[u][mp][r], a[mp][r]);
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    a[0][r] -= lam * a[1][r];
    ss = fmaf(a[0][r], a[0][r], ss);
  }
  ss = warp_sum(ss);
  const float k = post / sqrtf(ss / (float)dv + eps);
  bf16* orow = out + (size_t)t * ld_out + (size_t)h * dv;
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const int i = lane + 32 * r;
    if (i < dv) orow[i] = __float2bfloat16_rn(a[0][r] * k);
  }
}

// Into how many bfloat16 terms a softmax weight is split for the product with the values: 3 (all 24 bits: the weights are
// 32-bit in that product), or 1 with QORVIX_DIFF_WEIGHT_TERMS=1 (rounded to bfloat16 as in the other attention kernels;
// for comparison).
static inline int diff_weight_terms() {
  static int v = 0;
  if (!v) {
    const char* e = getenv("QORVIX_DIFF_WEIGHT_TERMS");
    v = (e && e[0] == '1') ? 1 : 3;
  }
  return v;
}

static inline int diff_pad_n(int n) { return n <= 32 ? 32 : (n <= 64 ? 64 : 128); }
static inline int diff_pad_dv(int dv) { return dv <= 64 ? 64 : (dv <= 128 ? 128 : 256); }

// Floats of workspace per (token, head, slice) of single tokens whose keys are cut into slices.
extern "C" long long qv_diff_partial_floats(int dv) { return 2LL * (diff_pad_dv(dv) + 2); }

// S segments starting at rows seg_q_start[s] of q/out (and of the step), the longest of max_q_len rows.  With max_q_len == 1
// and at most 16 query heads per key/value head the heads of a group share a tile (the keys are read once for them) and
// splits > 1 cuts every token's keys into that many slices: `partial` (S * H * splits * qv_diff_partial_floats floats) then
// holds what the merge finishes.  Refuses (QV_ERR_UNSUPPORTED, nothing written) sizes it does not take: map sizes above
// 128 or value sizes above 256, sizes that are no multiple of 8, rows that do not start on 16 bytes.
extern "C" int qv_diff_attention_tc(void* out, int ld_out, const void* q, int ld_q, const void* cache, const int* seg_q_start,
                                    const int* seg_pos0, const int* block_table, int max_blocks, int S, int max_q_len, int H, int G, int n,
                                    int dv, int page, int window, float scale, float lam, float eps, float post, float* partial, int splits,
                                    void* stream) {
  if (S <= 0 || max_q_len <= 0) return 0;
  if (n <= 0 || n > 128 || (n & 7) || dv <= 0 || dv > 256 || (dv & 7) || G <= 0 || H % G || (ld_q & 7) || (ld_out & 1) || page <= 0) return QV_ERR_UNSUPPORTED;
  if ((((uintptr_t)q | (uintptr_t)cache) & 15) || ((uintptr_t)out & 3) || ((G * (2 * n + dv)) & 7)) return QV_ERR_UNSUPPORTED;
  const bool grouped = max_q_len == 1 && H / G <= 16;
  if (splits > 1 && (!grouped || !partial || splits > 32)) return QV_ERR_UNSUPPORTED;
  if (S > 65535 || H > 65535) return QV_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const int NT = diff_pad_n(n), DVT = diff_pad_dv(dv);
  const bool small = max_q_len <= 16;
  const int MW = small ? 1 : 4;
  // four stages of 32 keys (the widest sizes: 169 KB, one CTA an SM, which their registers allow anyway); the ring must
  // also hold map 2's float32 rows at the end
  const size_t stage_bytes = (size_t)DIFF_KB * (2 * NT + 8 + DVT + 8) * sizeof(bf16), q_bytes = (size_t)(16 * MW) * (2 * NT + 8) * sizeof(bf16);
  constexpr int stages = 4;
  const size_t rows_bytes = (size_t)(16 * MW) * (DVT + 1) * sizeof(float);
  const size_t smem = q_bytes + (stages * stage_bytes > rows_bytes ? stages * stage_bytes : rows_bytes);
  const float scale_log2 = scale * 1.4426950408889634f;
  int page_shift = -1;
  if ((page & (page - 1)) == 0) for (page_shift = 0; (1 << page_shift) < page; ++page_shift) {}
  if (splits < 1) splits = 1;
  const int tiles = (max_q_len + 16 * MW - 1) / (16 * MW);
  if (!grouped && tiles > 65535) return QV_ERR_TOO_LARGE;
  const dim3 grid(grouped ? splits : H, S, grouped ? G : tiles);
  int rc = QV_ERR_UNSUPPORTED;
#define DIFF_LAUNCH_PT(N_, DV_, MW_, GR_, PT_)                                                                                      \
  do {                                                                                                                              \
    cudaFuncSetAttribute(diff_attention_tc_kernel<N_, DV_, MW_, GR_, stages, PT_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    rc = qv_launch(diff_attention_tc_kernel<N_, DV_, MW_, GR_, stages, PT_>, grid, dim3(MW_ == 1 ? 128 : 64 * MW_), smem, st, (bf16*)out, \
                   ld_out, (const bf16*)q, ld_q, (const bf16*)cache, seg_q_start, seg_pos0, block_table, max_blocks, H, G, n, dv,   \
                   page, page_shift, window, scale_log2, lam, eps, post, partial, splits);                                          \
  } while (0)
#define DIFF_LAUNCH(N_, DV_, MW_, GR_) do { if (diff_weight_terms() == 1) DIFF_LAUNCH_PT(N_, DV_, MW_, GR_, 1); else DIFF_LAUNCH_PT(N_, DV_, MW_, GR_, 3); } while (0)
#define DIFF_BY_MW(N_, DV_)                                                   \
  do {                                                                        \
    if (grouped) DIFF_LAUNCH(N_, DV_, 1, true);                               \
    else if (small) DIFF_LAUNCH(N_, DV_, 1, false);                           \
    else DIFF_LAUNCH(N_, DV_, 4, false);                                      \
  } while (0)
#define DIFF_BY_DV(N_) do { if (DVT == 64) DIFF_BY_MW(N_, 64); else if (DVT == 128) DIFF_BY_MW(N_, 128); else DIFF_BY_MW(N_, 256); } while (0)
  if (NT == 32) DIFF_BY_DV(32); else if (NT == 64) DIFF_BY_DV(64); else DIFF_BY_DV(128);
#undef DIFF_BY_DV
#undef DIFF_BY_MW
#undef DIFF_LAUNCH
#undef DIFF_LAUNCH_PT
  if (rc || splits <= 1) return rc;
  const int T = S;                                        // single tokens: a segment is a token
  const dim3 mgrid((T * H + 3) / 4);
  if (DVT == 64) return qv_launch(diff_merge_kernel<64>, mgrid, dim3(128), 0, st, (bf16*)out, ld_out, (const float*)partial, T, H, dv, splits, lam, eps, post);
  if (DVT == 128) return qv_launch(diff_merge_kernel<128>, mgrid, dim3(128), 0, st, (bf16*)out, ld_out, (const float*)partial, T, H, dv, splits, lam, eps, post);
  return qv_launch(diff_merge_kernel<256>, mgrid, dim3(128), 0, st, (bf16*)out, ld_out, (const float*)partial, T, H, dv, splits, lam, eps, post);
}
