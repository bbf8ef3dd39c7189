// Tensor-core attention over cached [key | value] rows whose key and value sizes may differ and whose scores may
// be shaped on their way to the softmax, for bfloat16 steps that carry runs of query tokens.
//
// A block owns a tile of 64 or 128 query rows: consecutive tokens of one request times the (padded) group of query
// heads that share one key/value head.  It walks the request's keys in tiles of 64 (first the tiles that hold kept
// first keys, then the window's), gathers the rows through the block table with 16-byte cp.async copies into
// swizzled shared memory (two tiles in flight), and runs scores and the weighted sum of values on mma.sync m16n8k16
// (bfloat16 in, float32 out).  Between the two products every score passes, in float32,
//     s = (q . k) * scale;  s *= head_scale[h];  s = cap * tanh(s / cap);  s -= slope[h] * (i - j)
// (each step optional), the mask (j <= i and (i - j < window or j < keep_first); or, by blocks of positions counted
// from the sequence's start, j <= i and i / chunk == j / chunk) and the running max/sum softmax, whose denominator may
// count a learned score per head once, without a value; the result may be multiplied by the sigmoid of a gate.
// Key size dk and value size dv are multiples of 8 up to 128; the tiles are padded with zeros to the next of
// 64 / 128 (keys) and 32 / 64 / 128 (values), which changes no sum.
#include "common.cuh"
#include "mma_sync.cuh"
#include "score_shape.cuh"

#include <math_constants.h>

namespace {

using namespace kvb_mma;

constexpr int BN = 64;   // keys per tile
constexpr float kLog2e = 1.4426950408889634f;

struct TileDesc { int req, t0, n_tok, pad; };

struct RowsArgs {
  const __nv_bfloat16* q; int q_row_stride;          // [T, >= nq * dk]
  const __nv_bfloat16* pages;                        // [num_pages, nkv, page_size, dk + dv]
  const int* block_table; int max_pages, page_shift, num_pages;
  const int* positions; const TileDesc* tiles;
  __nv_bfloat16* out;                                // [T, nq * dv]
  int nq, nkv, G, gp_shift, dk, dv;
  float scale; int window, keep_first, one_more;
  ScoreShape shape;
  int* status;
};

// KS: k-steps of 16 key channels (the padded key size is KS * 16); DP: pairs of 8 value channels (the padded
// value size is DP * 16); NW: warps, 16 query rows each.
template <int KS, int DP, int NW>
__global__ void __launch_bounds__(NW * 32)
window_flash_attention_kernel(RowsArgs p) {
  constexpr int BM = NW * 16;
  constexpr int kThreads = NW * 32;
  constexpr int KC = KS * 2, VC = DP * 2;                 // 16-byte chunks of a padded key / value row
  constexpr int PK = (KC + 7) / 8 * 128, PV = (VC + 7) / 8 * 128;      // bytes from row to row in shared memory
  constexpr int DT = DP * 2;                              // n-tiles of the output
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                              // [BM] rows of PK bytes
  unsigned char* k_s = q_s + BM * PK;                     // [2][BN] rows of PK bytes
  unsigned char* v_s = k_s + 2 * BN * PK;                 // [2][BN] rows of PV bytes
  int* row_pos = reinterpret_cast<int*>(v_s + 2 * BN * PV);            // [BM] position of each row's token, -1 if none

  pdl_trigger();
  pdl_wait();
  // the last tiles of a request read the most keys: they start first
  const TileDesc tile = p.tiles[gridDim.x - 1 - blockIdx.x];
  const int hk = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.G, gp_shift = p.gp_shift, gp = 1 << gp_shift;
  const int page_mask = (1 << p.page_shift) - 1;
  const int* table = p.block_table + (size_t)tile.req * p.max_pages;
  const int dk = p.dk, dv = p.dv, row_len = dk + dv, window = p.window;

  if (tid < BM) {
    const int ti = tid >> gp_shift, hi = tid & (gp - 1);
    row_pos[tid] = (ti < tile.n_tok && hi < G) ? p.positions[tile.t0 + ti] : -1;
  }
  const int pos_first = p.positions[tile.t0];
  const int pos_last = p.positions[tile.t0 + tile.n_tok - 1];
  const int k_hi = pos_last + 1;                                    // keys [.., k_hi) are read
  const int k_lo = first_seen_key(pos_first, window, p.shape.chunk);    // positions ascend: no row of the tile sees less
  const int first_tile = k_lo / BN, last_tile = (k_hi - 1) / BN;
  const int keep = window > 0 ? p.keep_first : 0;
  const int keep_tiles = min((keep + BN - 1) / BN, first_tile);
  const int n_walk = keep_tiles + last_tile - first_tile + 1;
  auto tile_at = [&](int idx) { return idx < keep_tiles ? idx : first_tile + idx - keep_tiles; };

  // ---- loaders ------------------------------------------------------------------
  auto load_q = [&]() {
    for (int c = tid; c < BM * KC; c += kThreads) {
      const int row = c / KC, part = c - row * KC;
      const int ti = row >> gp_shift, hi = row & (gp - 1);
      const bool ok = ti < tile.n_tok && hi < G && part * 8 < dk;
      const __nv_bfloat16* src = p.q + (size_t)(tile.t0 + (ok ? ti : 0)) * p.q_row_stride +
                                 (size_t)(hk * G + (ok ? hi : 0)) * dk + (ok ? part * 8 : 0);
      cp_async_16_zfill(q_s + swz_pitch<PK>(row, part), src, ok);
    }
  };
  // A key's row [key | value] is copied by kThreads / BN threads, so that its page is looked up once per thread and tile.
  auto load_kv = [&](int t, int buf) {
    constexpr int TPK = kThreads / BN;
    unsigned char* kd = k_s + buf * BN * PK;
    unsigned char* vd = v_s + buf * BN * PV;
    const int key = tid / TPK, sub = tid % TPK;
    const int j = t * BN + key;
    bool ok = j < k_hi && (j >= k_lo || j < keep);
    size_t off = 0;
    if (ok) {
      const int lp = j >> p.page_shift;
      const int page = lp < p.max_pages ? __ldg(table + lp) : -1;
      if (page < 0 || page >= p.num_pages) {
        atomicCAS(p.status, 0, KVB_STATUS_UNMAPPED_PAGE);
        ok = false;
      } else {
        off = ((((size_t)page * p.nkv + hk) << p.page_shift) + (j & page_mask)) * row_len;
      }
    }
#pragma unroll
    for (int c = sub; c < KC; c += TPK) {
      const bool have = ok && c * 8 < dk;
      cp_async_16_zfill(kd + swz_pitch<PK>(key, c), p.pages + off + (have ? c * 8 : 0), have);
    }
#pragma unroll
    for (int c = sub; c < VC; c += TPK) {
      const bool have = ok && c * 8 < dv;
      cp_async_16_zfill(vd + swz_pitch<PV>(key, c), p.pages + off + (have ? dk + c * 8 : 0), have);
    }
  };

  load_q();
  load_kv(tile_at(0), 0);
  cp_async_commit();

  // ---- per-thread state: rows r0 = warp*16 + lane/4 and r0 + 8 ---------------------
  float o[DT][4];
#pragma unroll
  for (int n = 0; n < DT; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};
  unsigned qf[KS][4];
  const int r0 = warp * 16 + (lane >> 2);
  int pos_r[2], lo_r[2];
  float hs[2], slope[2];             // the two rows' heads: factor on the score, slope of the distance bias
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int hi = (r0 + rr * 8) & (gp - 1);
    const int head = hk * G + (hi < G ? hi : 0);
    hs[rr] = p.scale * (p.shape.head_scale != nullptr ? p.shape.head_scale[head] : 1.f);
    slope[rr] = p.shape.slopes != nullptr ? p.shape.slopes[head] : 0.f;
  }
  const float cap = p.shape.softcap, inv_cap = cap > 0.f ? 1.0f / cap : 0.f;

  for (int idx = 0; idx < n_walk; ++idx) {
    const int t = tile_at(idx);
    const int buf = idx & 1;
    if (idx + 1 < n_walk) {
      load_kv(tile_at(idx + 1), buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (idx == 0) {
      // query fragments stay in registers for the whole walk
#pragma unroll
      for (int kk = 0; kk < KS; ++kk)
        ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3],
                    q_s + swz_pitch<PK>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));
      pos_r[0] = row_pos[r0]; pos_r[1] = row_pos[r0 + 8];
      lo_r[0] = first_seen_key(pos_r[0], window, p.shape.chunk);
      lo_r[1] = first_seen_key(pos_r[1], window, p.shape.chunk);
    }
    const unsigned char* kt = k_s + buf * BN * PK;
    const unsigned char* vt = v_s + buf * BN * PV;

    // S = Q K^T : 16 rows x 64 keys per warp
    float s[BN / 8][4];
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        unsigned b0, b1, b2, b3;
        // lanes 0-7: keys np*16+l, chunk 2kk | 8-15: same keys, chunk 2kk+1 | 16-23: keys +8, chunk 2kk | 24-31: keys +8, chunk 2kk+1
        const int key = np * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int chunk = kk * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(b0, b1, b2, b3, kt + swz_pitch<PK>(key, chunk));
        mma_bf16(s[2 * np], qf[kk], b0, b1);
        mma_bf16(s[2 * np + 1], qf[kk], b2, b3);
      }
    }
    // shape, mask and running softmax; from here on the scores are in units of log2
    const int kbase = t * BN + ((lane & 3) << 1);
    float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = kbase + n * 8 + (e & 1);
        const int rr = e >> 1;
        const bool ok = j <= pos_r[rr] && (j >= lo_r[rr] || j < keep);
        float v = s[n][e] * hs[rr];
        if (cap > 0.f) v = cap * tanhf(v * inv_cap);
        v = fmaf(-slope[rr], (float)(pos_r[rr] - j), v);
        s[n][e] = ok ? v * kLog2e : -CUDART_INF_F;
        mx[rr] = fmaxf(mx[rr], s[n][e]);
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
      const float m_new = fmaxf(m_run[rr], mx[rr]);
      m_use[rr] = (m_new == -CUDART_INF_F) ? 0.f : m_new;   // a row with no key yet: keep everything at zero
      corr[rr] = (m_run[rr] == -CUDART_INF_F) ? 0.f : exp2f(m_run[rr] - m_use[rr]);
      m_run[rr] = m_new;
      l_run[rr] *= corr[rr];
    }
#pragma unroll
    for (int n = 0; n < DT; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
    unsigned pf[BN / 16][4];
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
      const float p0 = exp2f(s[n][0] - m_use[0]), p1 = exp2f(s[n][1] - m_use[0]);
      const float p2 = exp2f(s[n][2] - m_use[1]), p3 = exp2f(s[n][3] - m_use[1]);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      // the accumulator layout of two neighbouring score tiles is the A layout of one k-step
      pf[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
      for (int dp = 0; dp < DP; ++dp) {
        unsigned b0, b1, b2, b3;
        // lanes 0-7: keys kk*16+l, chunk 2dp | 8-15: keys +8, chunk 2dp | 16-23: keys kk*16+l, chunk 2dp+1 | 24-31: keys +8, chunk 2dp+1
        const int key = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int chunk = dp * 2 + (lane >> 4);
        ldmatrix_x4_trans(b0, b1, b2, b3, vt + swz_pitch<PV>(key, chunk));
        mma_bf16(o[2 * dp], pf[kk], b0, b1);
        mma_bf16(o[2 * dp + 1], pf[kk], b2, b3);
      }
    }
    __syncthreads();  // the buffer just read is filled again by the next iteration's prefetch
  }

  // ---- normalise and store ---------------------------------------------------------
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
    l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int row = r0 + rr * 8;
    const int ti = row >> gp_shift, hi = row & (gp - 1);
    if (ti >= tile.n_tok || hi >= G) continue;
    if (p.one_more)      // the one more key: score 0, which is 0 in units of log2 too; no value
      l_run[rr] += (m_run[rr] == -CUDART_INF_F) ? 1.f : exp2f(-m_run[rr]);
    if (p.shape.sinks != nullptr) {     // the head's learned score, in units of log2 like the running maximum
      const float sink = p.shape.sinks[hk * G + hi] * kLog2e;
      if (m_run[rr] == -CUDART_INF_F) {
        l_run[rr] = 1.f;
      } else if (sink - m_run[rr] > 100.f) {     // the sink outweighs every key beyond what a float holds: nothing is left
        l_run[rr] = CUDART_INF_F;
      } else {
        l_run[rr] += exp2f(sink - m_run[rr]);
      }
    }
    const float inv = (l_run[rr] > 0.f && l_run[rr] < CUDART_INF_F) ? p.shape.out_scale / l_run[rr] : 0.f;
    const size_t at = ((size_t)(hk * G + hi)) * dv + ((lane & 3) << 1);
    __nv_bfloat16* dst = p.out + (size_t)(tile.t0 + ti) * p.nq * dv + at;
    const __nv_bfloat16* gate = p.shape.gate != nullptr
        ? static_cast<const __nv_bfloat16*>(p.shape.gate) + (size_t)(tile.t0 + ti) * p.shape.gate_ld + at : nullptr;
#pragma unroll
    for (int n = 0; n < DT; ++n)
      if (n * 8 + ((lane & 3) << 1) < dv) {
        float a = o[n][rr * 2] * inv, b = o[n][rr * 2 + 1] * inv;
        if (gate != nullptr) {
          a *= 1.0f / (1.0f + expf(-__bfloat162float(gate[n * 8])));
          b *= 1.0f / (1.0f + expf(-__bfloat162float(gate[n * 8 + 1])));
        }
        *reinterpret_cast<unsigned*>(dst + n * 8) = pack_bf16(a, b);
      }
  }
}

template <int KS, int DP, int NW>
int launch(const RowsArgs& a, int num_tiles, cudaStream_t stream) {
  constexpr int BM = NW * 16;
  constexpr int PK = (KS * 2 + 7) / 8 * 128, PV = (DP * 2 + 7) / 8 * 128;
  const size_t smem = (size_t)BM * PK + 2 * (size_t)BN * (PK + PV) + BM * sizeof(int);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(window_flash_attention_kernel<KS, DP, NW>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  kvb_launch(window_flash_attention_kernel<KS, DP, NW>, dim3(num_tiles, a.nkv), dim3(NW * 32), smem, stream, a);
  return kvb_launch_result();
}

template <int KS, int NW>
int launch_dv(const RowsArgs& a, int num_tiles, cudaStream_t stream) {
  if (a.dv <= 32) return launch<KS, 2, NW>(a, num_tiles, stream);
  if (a.dv <= 64) return launch<KS, 4, NW>(a, num_tiles, stream);
  return launch<KS, 8, NW>(a, num_tiles, stream);
}

int log2_exact(int x) {
  int s = 0;
  while ((1 << s) < x) ++s;
  return (1 << s) == x ? s : -1;
}

}  // namespace

// 1 when the kernel takes these sizes: key and value sizes that are multiples of 8 up to 128, a group of at most
// 64 query heads per key/value head, a page size that is a power of two.
KVB_EXPORT int kvb_window_flash_attention_supported(int dk, int dv, int group, int page_size) {
  return dk >= 8 && dk <= 128 && dk % 8 == 0 && dv >= 8 && dv <= 128 && dv % 8 == 0 && group >= 1 && group <= 64 &&
         log2_exact(page_size) >= 0;
}

// tiles: num_tiles x {request row, first token row, tokens, 0}, int32; a tile holds consecutive tokens of one
// request, positions ascending, at most (wide ? 128 : 64) / (the group padded to a power of two) of them.
// q [T, >= nq * dk] with row stride q_row_stride; pages [num_pages, nkv, page_size, dk + dv]; out [T, nq * dv];
// all bfloat16, q and pages aligned to 16 bytes, q_row_stride a multiple of 8.  head_scale and slopes are
// float32 [nq] or null; softcap 0 for none; out_scale multiplies the result.  sinks: float32 [nq] or null; chunk: 0 or
// the size of the blocks of positions (not together with keep_first); gate: bfloat16 [T, >= nq * dv] with row stride
// gate_ld, or null.
KVB_EXPORT int kvb_window_flash_attention_masked(const void* q, int q_row_stride, const void* pages, const int* block_table,
                                                 int max_pages, int page_size, int num_pages, const int* positions,
                                                 const void* tiles, int num_tiles, int wide, void* out, int nq, int nkv,
                                                 int dk, int dv, float scale, int window, int keep_first, int one_more,
                                                 const float* head_scale, const float* slopes, float softcap,
                                                 float out_scale, const float* sinks, int chunk, const void* gate,
                                                 int gate_ld, int* status, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (nkv < 1 || nkv > 65535 || nq % nkv || window < 0 || keep_first < 0 || softcap < 0.f) return KVB_ERR_BAD_SIZE;
  if (chunk < 0 || (chunk > 0 && keep_first > 0) || (one_more && sinks != nullptr)) return KVB_ERR_BAD_SIZE;
  const int G = nq / nkv;
  if (!kvb_window_flash_attention_supported(dk, dv, G, page_size)) return KVB_ERR_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (q_row_stride & 7) || (reinterpret_cast<uintptr_t>(pages) & 15))
    return KVB_ERR_ALIGN;
  RowsArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q); a.q_row_stride = q_row_stride;
  a.pages = static_cast<const __nv_bfloat16*>(pages);
  a.block_table = block_table; a.max_pages = max_pages; a.page_shift = log2_exact(page_size); a.num_pages = num_pages;
  a.positions = positions; a.tiles = static_cast<const TileDesc*>(tiles);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.nq = nq; a.nkv = nkv; a.G = G; a.dk = dk; a.dv = dv;
  a.gp_shift = 0;
  while ((1 << a.gp_shift) < G) ++a.gp_shift;
  a.scale = scale; a.window = window; a.keep_first = keep_first; a.one_more = one_more;
  a.shape = ScoreShape{head_scale, slopes, softcap, out_scale, sinks, chunk, gate, gate_ld};
  a.status = status;
  if (dk <= 64) return wide ? launch_dv<4, 8>(a, num_tiles, stream) : launch_dv<4, 4>(a, num_tiles, stream);
  return wide ? launch_dv<8, 8>(a, num_tiles, stream) : launch_dv<8, 4>(a, num_tiles, stream);
}

KVB_EXPORT int kvb_window_flash_attention(const void* q, int q_row_stride, const void* pages, const int* block_table,
                                          int max_pages, int page_size, int num_pages, const int* positions,
                                          const void* tiles, int num_tiles, int wide, void* out, int nq, int nkv,
                                          int dk, int dv, float scale, int window, int keep_first, int one_more,
                                          const float* head_scale, const float* slopes, float softcap, float out_scale,
                                          int* status, cudaStream_t stream) {
  return kvb_window_flash_attention_masked(q, q_row_stride, pages, block_table, max_pages, page_size, num_pages, positions,
                                           tiles, num_tiles, wide, out, nq, nkv, dk, dv, scale, window, keep_first,
                                           one_more, head_scale, slopes, softcap, out_scale, nullptr, 0, nullptr, 0,
                                           status, stream);
}
