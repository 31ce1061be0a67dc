// Paged decode attention for 16-bit queries on sm_100a.
//
// Work decomposition: one CTA per (sequence, kv head, context range).  All query
// heads of the kv head's GQA group ride in the M dimension of warp-level
// m16n8k16 MMAs, so each KV block is fetched from HBM once per group instead of
// once per query head.  The reference launches one CTA per *query* head
// (src/kernels/src/pagedattention.cu:147-150, grid at :632 and :806) and walks K
// and V in two passes with dependent global loads (:200-246, :317-348).
//
// Data movement: for one (physical block, kv head) the K tile [HEAD/x][BS][x] and
// the V tile [HEAD][BS] are each one contiguous run of HEAD*BS elements
// (layouts: src/kernels/src/reshape_and_cache_kernel.cu:34-57).  Each warp owns a
// private ring of shared-memory stages and fills it with 1-D bulk async copies
// (cp.async.bulk, completion on an mbarrier), one copy per tile; no thread ever
// issues a per-element global load for KV data.  Warps never synchronise with
// each other inside the main loop; each keeps its own online-softmax state and
// the CTA merges the per-warp states once at the end.
//
// Fragment mapping (the part that is easy to get wrong):
//  * QK^T: A = Q (rows = query heads of the group, zero-padded to 16),
//    B = K with n = token.  The two n-tiles of a 16-token tile hold the tokens
//    {0,1,4,5,10,11,14,15} and {2,3,6,7,8,9,12,13}: every ldmatrix phase then
//    touches 8 distinct 16-byte bank groups, and lane quad-index q ends up with
//    the four logits of tokens 4q..4q+3.
//  * PV: A = P straight from those registers, B = V with k = token.  Because lane
//    q owns tokens 4q..4q+3 its B fragment is one 8-byte shared load from the V
//    row (16-bit cache) or one 4-byte word (FP8 cache), conflict-free.
//  * FP8 cache: the tiles feed m16n8k32 E4M3 MMAs directly (no per-element widening, which would
//    make the kernel instruction-bound).  The other operand is split in two FP8 terms so that
//    nothing is lost to its 3-bit mantissa: each query row is scaled to the E4M3 range and written
//    as head + tail (two MMAs per tile), and so are the probabilities (scaled by 2^8).  The row
//    scales, k_scale and v_scale are applied to the fp32 logits and the fp32 output.
#pragma once

#include <cooperative_groups.h>

#include <type_traits>

#include "pa_common.cuh"

namespace pa {

struct DecodeParams {
  void* out;              // [num_seqs, num_heads, HEAD], query dtype
  float* exp_sums;        // v2 scratch [num_seqs, num_heads, max_parts] (null: single pass)
  float* max_logits;      // v2 scratch [num_seqs, num_heads, max_parts]
  void* tmp_out;          // v2 scratch [num_seqs, num_heads, max_parts, HEAD], query dtype
  const void* q;          // [num_seqs, num_heads, HEAD], row stride q_stride
  const void* k_cache;
  const void* v_cache;
  const uint32_t* block_tables;
  const uint32_t* context_lens;
  const float* alibi_slopes;  // may be null
  unsigned* status;
  int64_t kv_block_stride;    // elements
  int64_t kv_head_stride;     // elements
  int num_seqs, num_heads, num_kv_heads, group;
  int max_num_blocks_per_seq, max_parts, q_stride;
  int partition_size;         // 0: the CTA (or cluster) covers the whole context
  int cluster;                // single pass only: CTAs per (sequence, kv head) that split the context (1 = one CTA)
  float scale, softcap, k_scale, v_scale;
};

template <typename T, bool FP8, int HEAD, int BS>
struct DecodeCfg {
  using MT = T;  // input type of the 16-bit MMAs (the FP8 path uses E4M3 MMAs instead)
  static constexpr int ES = FP8 ? 1 : 2;
#ifndef PA_STAGE_TOKENS_16BIT
#define PA_STAGE_TOKENS_16BIT 16
#endif
#ifndef PA_STAGE_TOKENS_FP8
#define PA_STAGE_TOKENS_FP8 32
#endif
  // Tokens per stage: at least one physical block and one 16-token MMA tile.  An FP8 stage takes 32
  // tokens so that it carries as many bytes, and as much independent work per warp, as a 16-bit one.
  static constexpr int STOK_MIN = FP8 ? PA_STAGE_TOKENS_FP8 : PA_STAGE_TOKENS_16BIT;
  static constexpr int SB = BS >= STOK_MIN ? 1 : STOK_MIN / BS;  // physical blocks per stage
  static constexpr int STOK = BS * SB;               // tokens per stage
  static constexpr int TT = STOK / 16;               // 16-token tiles per stage
  static constexpr int TILE_BYTES = HEAD * BS * ES;  // one block's K tile (V tile is the same size)
  static constexpr int STAGE_BYTES = 2 * SB * TILE_BYTES;
#ifdef PA_FORCE_NW
  static constexpr int NW = PA_FORCE_NW;
#else
  static constexpr int NW = STAGE_BYTES <= 12 * 1024 ? 4 : (STAGE_BYTES <= 16 * 1024 ? 3 : 2);
#endif
#ifdef PA_FORCE_STAGES
  static constexpr int STAGES = PA_FORCE_STAGES;
#else
  static constexpr int STAGES_RAW = (104 * 1024) / (NW * STAGE_BYTES);
  static constexpr int STAGES = STAGES_RAW < 2 ? 2 : (STAGES_RAW > 4 ? 4 : STAGES_RAW);
#endif
  static constexpr int THREADS = NW * WARP;
  static constexpr int RING_BYTES = NW * STAGES * STAGE_BYTES;
  static constexpr int ROW_F = HEAD + 8;  // padded fp32 row of the merge buffer
  static constexpr int WARP_MERGE_BYTES = NW * 16 * ROW_F * 4 + NW * 16 * 2 * 4;  // per-warp (acc, m, l)
  static constexpr int MERGE_BYTES = WARP_MERGE_BYTES + 16 * ROW_F * 4 + 16 * 2 * 4;  // + the CTA's own result (cluster mode)
  static constexpr int DATA_BYTES = RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES;
  static constexpr int BAR_BYTES = NW * STAGES * 2 * 8;
  static constexpr int SMEM_BYTES = DATA_BYTES + BAR_BYTES + 128;  // +128: manual alignment slack
  static_assert(HEAD % 16 == 0, "head size must be a multiple of 16");
  static_assert(!FP8 || (HEAD % 32 == 0 && BS >= 16), "FP8 path needs HEAD % 32 == 0 and block_size >= 16");
};

template <typename T, bool FP8, int HEAD, int BS>
__global__ void __launch_bounds__(DecodeCfg<T, FP8, HEAD, BS>::THREADS)
paged_decode_mma_kernel(const DecodeParams p) {
  using C = DecodeCfg<T, FP8, HEAD, BS>;
  using MT = typename C::MT;
  constexpr int NW = C::NW, STAGES = C::STAGES, SB = C::SB, STOK = C::STOK, TT = C::TT;
  constexpr int TILE_BYTES = C::TILE_BYTES, STAGE_BYTES = C::STAGE_BYTES;
  constexpr int KSTEPS = FP8 ? HEAD / 32 : HEAD / 16;  // MMA k-steps of QK^T
  constexpr int NT = HEAD / 8;       // n-tiles of PV

  namespace cg = cooperative_groups;
  constexpr int PART = PA_PARTITION_SIZE;   // the context is walked in chunks of this many tokens
  constexpr int SPC = PART / STOK;          // stages per full chunk
  static_assert(PART % STOK == 0 && SPC >= NW, "a chunk must hold at least one stage per warp");

  // Lets a dependent launch (the partition merge) be scheduled while this grid drains.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int seq = blockIdx.y;
  const int ctx = static_cast<int>(p.context_lens[seq]);
  const int gsplit = (p.group + 15) / 16;               // head sub-groups per kv head (1 unless group > 16)
  const int kvh = blockIdx.x / gsplit;
  const int head0 = kvh * p.group + (blockIdx.x % gsplit) * 16;
  const int nrows = min(16, kvh * p.group + p.group - head0);  // live rows of the M tile
  const bool rows16 = nrows > 8;
  const bool partitioned = p.partition_size > 0;
  const int csize = partitioned ? 1 : p.cluster;        // CTAs sharing this (sequence, kv head)
  const int part = blockIdx.z;                          // partition (v2) or rank in the cluster (v1)

  // Chunks of PART tokens owned by this CTA: first, first + cstride, ...  (v2: exactly one.)
  const int first = (partitioned || csize > 1) ? part : 0;
  const int cstride = partitioned ? (1 << 20) : csize;
  const int t_end = partitioned ? min(ctx, (first + 1) * PART) : ctx;
  const int nchunks_total = (t_end + PART - 1) / PART;
  const int my_chunks = first < nchunks_total ? (nchunks_total - 1 - first) / cstride + 1 : 0;
  if (csize == 1 && my_chunks == 0 && partitioned) return;  // nothing to do for this partition

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gi = lane >> 2, qi = lane & 3;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const uint32_t ring = smem_addr(smem) + warp * (STAGES * STAGE_BYTES);
  const uint32_t bars = smem_addr(smem) + C::DATA_BYTES + warp * (STAGES * 16);  // [stage]{K,V}

  if (ctx == 0 && csize == 1) {
    // Empty context: the reference's loops do not run and its accumulators stay zero.
    if (!partitioned) {
      T* o = reinterpret_cast<T*>(p.out) + (static_cast<int64_t>(seq) * p.num_heads + head0) * HEAD;
      for (int i = threadIdx.x; i < nrows * HEAD; i += C::THREADS) o[i] = from_f32<T>(0.f);
    }
    return;
  }

  if (lane == 0) {
    for (int s = 0; s < STAGES * 2; ++s) mbar_init(bars + s * 8, 1);
    mbar_init_fence();
  }
  __syncwarp();

  // ---- this warp's share: in every chunk of the CTA, stages warp, warp + NW, ...
  const int cnt_full = (SPC - warp + NW - 1) / NW;      // this warp's stages in a full chunk
  int n_mine = 0;
  if (my_chunks > 0) {
    const int lc = first + (my_chunks - 1) * cstride;   // the CTA's last chunk; only it can be short
    const int lsc = (min(t_end, (lc + 1) * PART) - lc * PART + STOK - 1) / STOK;
    n_mine = (my_chunks - 1) * cnt_full + (lsc > warp ? (lsc - warp + NW - 1) / NW : 0);
  }
  // First token of this warp's local stage (k-th chunk of the CTA, j-th stage of the warp in it).
  auto tok0_of = [&](int k, int j) { return (first + k * cstride) * PART + (warp + j * NW) * STOK; };
  const int last_block = ctx > 0 ? (ctx - 1) / BS : 0;  // last block-table slot of the sequence that holds tokens
  const uint32_t* table = p.block_tables + static_cast<int64_t>(seq) * p.max_num_blocks_per_seq;
  const int64_t head_off = static_cast<int64_t>(kvh) * p.kv_head_stride;
  const unsigned char* kc = reinterpret_cast<const unsigned char*>(p.k_cache);
  const unsigned char* vc = reinterpret_cast<const unsigned char*>(p.v_cache);
  const uint64_t policy = policy_evict_first();

  // Block-table entries for a window of 32 of this warp's stages live one per lane.
  auto load_entries = [&](int round, uint32_t (&e)[SB]) {
    const int i = round * 32 + lane;
    const int k = min(i / cnt_full, max(my_chunks - 1, 0));
    const int slot0 = tok0_of(k, i - k * cnt_full) / BS;
#pragma unroll
    for (int b = 0; b < SB; ++b) e[b] = (i < n_mine && slot0 + b <= last_block) ? table[slot0 + b] : 0xffffffffu;
  };
  uint32_t ent_cur[SB], ent_nxt[SB];
  load_entries(0, ent_cur);
  load_entries(1, ent_nxt);
  int ent_round = 0;  // round held by ent_cur

  // Issues the copies of local stage i (all lanes call; lane 0 issues).
  auto issue = [&](int i) {
    const int r = i >> 5;
    uint32_t e[SB];
    if (r == ent_round) {  // warp-uniform; keeps the younger window's load off this path
#pragma unroll
      for (int b = 0; b < SB; ++b) e[b] = __shfl_sync(0xffffffffu, ent_cur[b], i & 31);
    } else {
#pragma unroll
      for (int b = 0; b < SB; ++b) e[b] = __shfl_sync(0xffffffffu, ent_nxt[b], i & 31);
    }
    if (lane == 0) {
      const int s = i % STAGES;
      const uint32_t dst = ring + s * STAGE_BYTES;
      const uint32_t bk = bars + s * 16, bv = bk + 8;
      int nb = 0;
#pragma unroll
      for (int b = 0; b < SB; ++b) nb += (e[b] != 0xffffffffu);
      mbar_expect_tx(bk, nb * TILE_BYTES);
#pragma unroll
      for (int b = 0; b < SB; ++b)
        if (e[b] != 0xffffffffu)
          bulk_g2s(dst + b * TILE_BYTES, kc + (static_cast<int64_t>(e[b]) * p.kv_block_stride + head_off) * C::ES,
                   TILE_BYTES, bk, policy);
      mbar_expect_tx(bv, nb * TILE_BYTES);
#pragma unroll
      for (int b = 0; b < SB; ++b)
        if (e[b] != 0xffffffffu)
          bulk_g2s(dst + (SB + b) * TILE_BYTES, vc + (static_cast<int64_t>(e[b]) * p.kv_block_stride + head_off) * C::ES,
                   TILE_BYTES, bv, policy);
    }
  };

  // Prologue: fill the ring.
#pragma unroll
  for (int i = 0; i < STAGES; ++i)
    if (i < n_mine) issue(i);

  // ---- query fragments (A operand), zero rows beyond the group
  // 16-bit path: qa[j] = the four A registers of k-step j.  FP8 path: qa = head terms, qb = tail terms,
  // and qinv_* undo the per-row scaling that brought the row into the E4M3 range.
  uint32_t qa[KSTEPS][4];
  uint32_t qb[FP8 ? KSTEPS : 1][4];
  float qinv_lo = 1.f, qinv_hi = 1.f;
  {
    const T* qbase = reinterpret_cast<const T*>(p.q) + static_cast<int64_t>(seq) * p.q_stride + static_cast<int64_t>(head0) * HEAD;
    if constexpr (!FP8) {
      auto ldq = [&](int row, int col) -> uint32_t {  // two consecutive elements
        return row < nrows ? *reinterpret_cast<const uint32_t*>(qbase + row * HEAD + col) : 0u;
      };
#pragma unroll
      for (int j = 0; j < KSTEPS; ++j) {
        qa[j][0] = ldq(gi, 16 * j + 2 * qi);
        qa[j][1] = ldq(gi + 8, 16 * j + 2 * qi);
        qa[j][2] = ldq(gi, 16 * j + 8 + 2 * qi);
        qa[j][3] = ldq(gi + 8, 16 * j + 8 + 2 * qi);
      }
      (void)qb;
    } else {
      // This lane's 4-element runs of rows gi and gi + 8: dims 32j + 4q.. and 32j + 16 + 4q..
      // Two passes over the (tiny, cached) query rows keep the register footprint small: the first finds
      // each row's largest magnitude, the second scales and splits.
      auto load4 = [&](int j, int reg, float (&v)[4]) {
        const int row = gi + (reg & 1) * 8, col = 32 * j + (reg >> 1) * 16 + 4 * qi;
        uint2 raw = make_uint2(0u, 0u);
        if (row < nrows) {
          raw.x = *reinterpret_cast<const uint32_t*>(qbase + row * HEAD + col);
          raw.y = *reinterpret_cast<const uint32_t*>(qbase + row * HEAD + col + 2);
        }
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = to_f32<T>(e[k]);
      };
      float amax_lo = 0.f, amax_hi = 0.f;
#pragma unroll
      for (int j = 0; j < KSTEPS; ++j) {
#pragma unroll
        for (int reg = 0; reg < 4; ++reg) {
          float v[4];
          load4(j, reg, v);
          const float m4 = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
          if (reg & 1) amax_hi = fmaxf(amax_hi, m4);
          else amax_lo = fmaxf(amax_lo, m4);
        }
      }
      amax_lo = fmaxf(amax_lo, __shfl_xor_sync(0xffffffffu, amax_lo, 1));
      amax_lo = fmaxf(amax_lo, __shfl_xor_sync(0xffffffffu, amax_lo, 2));
      amax_hi = fmaxf(amax_hi, __shfl_xor_sync(0xffffffffu, amax_hi, 1));
      amax_hi = fmaxf(amax_hi, __shfl_xor_sync(0xffffffffu, amax_hi, 2));
      // Scale the row so that its largest element sits at 224 (half the E4M3 maximum).
      const float qs_lo = amax_lo > 0.f && amax_lo < 3.0e38f ? 224.f / amax_lo : 1.f;
      const float qs_hi = amax_hi > 0.f && amax_hi < 3.0e38f ? 224.f / amax_hi : 1.f;
      qinv_lo = 1.f / qs_lo;
      qinv_hi = 1.f / qs_hi;
#pragma unroll
      for (int j = 0; j < KSTEPS; ++j) {
#pragma unroll
        for (int reg = 0; reg < 4; ++reg) {
          float v[4];
          load4(j, reg, v);
          const float sc = (reg & 1) ? qs_hi : qs_lo;
          uint32_t h01, t01, h23, t23;
          split_e4m3x2(v[0] * sc, v[1] * sc, h01, t01);
          split_e4m3x2(v[2] * sc, v[3] * sc, h23, t23);
          qa[j][reg] = h01 | (h23 << 16);
          qb[j][reg] = t01 | (t23 << 16);
        }
      }
    }
  }

  // ---- per-lane shared-memory offsets
  // K (ldmatrix row addresses).  Matrix mi = lane / 8, row r = lane % 8.
  uint32_t koff[TT];
  {
    const int mi = lane >> 3, r = lane & 7;
    const int tile = mi >> 1;     // which n-tile this matrix feeds
    const int chunk = mi & 1;     // which 16-byte chunk of the k-step
    const int tau = 4 * (r >> 1) + (r & 1) + ((((r >> 2) ^ tile) & 1) ? 2 : 0);
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      const int ts = tt * 16 + tau;
      koff[tt] = (ts / BS) * TILE_BYTES + (chunk * BS + (ts % BS)) * 16;
    }
  }
  // V.  16-bit: one 8-byte load per n-tile at row gi.  FP8: ldmatrix rows; one x4 load brings, for two
  // n-tiles, the 16-byte halves that hold stage tokens 0-15 and 16-31 (voff8: matrix mi = lane / 8 serves
  // n-tile mi / 2, half mi % 2).
  uint32_t voff[TT];
  uint32_t voff8 = 0;
  if constexpr (FP8) {
    static_assert(!FP8 || TT == 2, "the FP8 path walks 32-token stages");
    const int mi = lane >> 3, r = lane & 7, half = mi & 1;
    const int vb = (half * 16) / BS, vo = (half * 16) % BS;
    voff8 = (SB + vb) * TILE_BYTES + ((mi >> 1) * 8 + r) * BS + vo;
  }
#pragma unroll
  for (int tt = 0; tt < TT; ++tt) {
    const int vb = (tt * 16) / BS, vo = (tt * 16) % BS;  // block within the stage and token offset in it
    if constexpr (FP8) {
      voff[tt] = 0;
    } else if constexpr (BS >= 16) {
      voff[tt] = (SB + vb) * TILE_BYTES + (gi * BS + vo + 4 * qi) * 2;
    } else {
      voff[tt] = (SB + 2 * tt + (qi >> 1)) * TILE_BYTES + (gi * BS + (qi & 1) * 4) * 2;
    }
  }
  // Tokens (within a 16-token tile) behind this lane's logits: n-tile 0 -> tokA, tokA+1; n-tile 1 -> tokB, tokB+1.
  const int tokA = 4 * qi + ((qi & 2) ? 2 : 0);
  const int tokB = 4 * qi + ((qi & 2) ? 0 : 2);

  // ---- softmax state (log2 domain) and output accumulators
  const bool plain = (p.softcap == 1.0f) && (p.alibi_slopes == nullptr);
  const float kscale = FP8 ? p.k_scale : 1.0f;
  const float qk_scale = p.scale * kscale;
  const float qk_scale_log2 = qk_scale * LOG2E;
  float slope_lo = 0.f, slope_hi = 0.f;
  if (p.alibi_slopes != nullptr) {
    if (gi < nrows) slope_lo = p.alibi_slopes[head0 + gi];
    if (gi + 8 < nrows) slope_hi = p.alibi_slopes[head0 + gi + 8];
  }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;

  bool healthy = true;
  int ck = 0, cj = 0;  // chunk ordinal and stage-within-chunk of local stage i

  for (int i = 0; i < n_mine && healthy; ++i) {
    const int s = i % STAGES;
    const uint32_t par = (i / STAGES) & 1;
    const uint32_t stage = ring + s * STAGE_BYTES;
    const uint32_t bk = bars + s * 16, bv = bk + 8;
    const int stage_tok0 = tok0_of(ck, cj);
    if (++cj == cnt_full) { cj = 0; ++ck; }

    // Rotate the block-table window when the stage to be issued this iteration enters a new round.
    if (((i + STAGES) >> 5) > ent_round + 1) {
#pragma unroll
      for (int b = 0; b < SB; ++b) ent_cur[b] = ent_nxt[b];
      ++ent_round;
      load_entries(ent_round + 1, ent_nxt);
    }

    healthy = __all_sync(0xffffffffu, mbar_wait(bk, par, p.status));
    if (!healthy) break;

#ifdef PA_DEBUG_SKIP_COMPUTE
    // Measurement aid (never defined in a product build): stream the tiles and do no arithmetic, which
    // gives the bandwidth ceiling of this access pattern.
    healthy = __all_sync(0xffffffffu, mbar_wait(bv, par, p.status));
    if (!healthy) break;
    __syncwarp();
    if (i + STAGES < n_mine) issue(i + STAGES);
    continue;
#endif
    // ---------------- logits of the stage's tiles (independent MMA chains: they overlap)
    float sc[TT][2][4];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
#pragma unroll
      for (int h = 0; h < 2; ++h) sc[tt][h][0] = sc[tt][h][1] = sc[tt][h][2] = sc[tt][h][3] = 0.f;
    }
    if constexpr (!FP8) {
#pragma unroll
      for (int j = 0; j < KSTEPS; ++j) {
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
          if (TT == 1 || stage_tok0 + tt * 16 < t_end) {
            uint32_t r0, r1, r2, r3;
            ldmatrix_x4(stage + koff[tt] + j * (2 * BS * 16), r0, r1, r2, r3);
            mma16816<MT>(sc[tt][0], qa[j][0], qa[j][1], qa[j][2], qa[j][3], r0, r1);
            mma16816<MT>(sc[tt][1], qa[j][0], qa[j][1], qa[j][2], qa[j][3], r2, r3);
          }
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < KSTEPS; ++j) {
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
          if (stage_tok0 + tt * 16 < t_end) {
            uint32_t r0, r1, r2, r3;
            ldmatrix_x4(stage + koff[tt] + j * (2 * BS * 16), r0, r1, r2, r3);
            mma16832_e4m3(sc[tt][0], qa[j][0], qa[j][1], qa[j][2], qa[j][3], r0, r1);
            mma16832_e4m3(sc[tt][1], qa[j][0], qa[j][1], qa[j][2], qa[j][3], r2, r3);
            mma16832_e4m3(sc[tt][0], qb[j][0], qb[j][1], qb[j][2], qb[j][3], r0, r1);
            mma16832_e4m3(sc[tt][1], qb[j][0], qb[j][1], qb[j][2], qb[j][3], r2, r3);
          }
        }
      }
    }

    // ---------------- online softmax over the whole stage (one max / one rescale per stage)
    // x[tt][0..3]: logits (log2 domain) of tokens tokA, tokA+1, tokB, tokB+1 of tile tt; -inf when masked.
    auto logits_of = [&](int rowsel, float slope, float rowscale, float (&x)[TT][4]) {
#pragma unroll
      for (int tt = 0; tt < TT; ++tt) {
        const int ta = stage_tok0 + tt * 16 + tokA, tb = stage_tok0 + tt * 16 + tokB;
        float x0 = sc[tt][0][rowsel], x1 = sc[tt][0][rowsel + 1], x2 = sc[tt][1][rowsel], x3 = sc[tt][1][rowsel + 1];
        if (plain) {
          const float f = qk_scale_log2 * rowscale;
          x0 *= f; x1 *= f; x2 *= f; x3 *= f;
        } else {
          const float f = qk_scale * rowscale;
          x0 *= f; x1 *= f; x2 *= f; x3 *= f;
          if (p.softcap != 1.0f) {
            const float inv = 1.0f / p.softcap;
            x0 = tanh_approx(x0 * inv) * p.softcap; x1 = tanh_approx(x1 * inv) * p.softcap;
            x2 = tanh_approx(x2 * inv) * p.softcap; x3 = tanh_approx(x3 * inv) * p.softcap;
          }
          x0 = (x0 + slope * static_cast<float>(ta - ctx + 1)) * LOG2E;
          x1 = (x1 + slope * static_cast<float>(ta + 1 - ctx + 1)) * LOG2E;
          x2 = (x2 + slope * static_cast<float>(tb - ctx + 1)) * LOG2E;
          x3 = (x3 + slope * static_cast<float>(tb + 1 - ctx + 1)) * LOG2E;
        }
        x[tt][0] = ta < t_end ? x0 : -INFINITY;
        x[tt][1] = ta + 1 < t_end ? x1 : -INFINITY;
        x[tt][2] = tb < t_end ? x2 : -INFINITY;
        x[tt][3] = tb + 1 < t_end ? x3 : -INFINITY;
      }
    };
    auto row_max = [&](const float (&x)[TT][4]) {
      float mx = -INFINITY;
#pragma unroll
      for (int tt = 0; tt < TT; ++tt) mx = fmaxf(mx, fmaxf(fmaxf(x[tt][0], x[tt][1]), fmaxf(x[tt][2], x[tt][3])));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      return fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    };
    // P fragments.  16-bit path: pa_*[tile][k-lo / k-hi]; lane q pairs tokens (4q, 4q+1) with V's low word and
    // (4q+2, 4q+3) with its high word.  FP8 path: pa_*[tile][head / tail], each register the four bytes of
    // tokens 4q..4q+3; probabilities carry a factor 2^8 (kPBias) that cancels between numerator and denominator.
    constexpr float kPBias = FP8 ? 8.f : 0.f;
    uint32_t pa_lo[TT][2], pa_hi[TT][2];
    auto probs = [&](const float (&x)[TT][4], float m, float& l, uint32_t (&pa)[TT][2]) {
      float sum = 0.f;
      const float mb = m - kPBias;
#pragma unroll
      for (int tt = 0; tt < TT; ++tt) {
        const float p0 = exp2_approx(x[tt][0] - mb), p1 = exp2_approx(x[tt][1] - mb);
        const float p2 = exp2_approx(x[tt][2] - mb), p3 = exp2_approx(x[tt][3] - mb);
        sum += (p0 + p1) + (p2 + p3);
        if constexpr (!FP8) {
          const uint32_t pA = pack2<MT>(p0, p1), pB = pack2<MT>(p2, p3);
          pa[tt][0] = (qi & 2) ? pB : pA;
          pa[tt][1] = (qi & 2) ? pA : pB;
        } else {
          uint32_t hA, tA, hB, tB;
          split_e4m3x2(p0, p1, hA, tA);   // tokens tokA, tokA + 1
          split_e4m3x2(p2, p3, hB, tB);   // tokens tokB, tokB + 1
          pa[tt][0] = (qi & 2) ? (hB | (hA << 16)) : (hA | (hB << 16));
          pa[tt][1] = (qi & 2) ? (tB | (tA << 16)) : (tA | (tB << 16));
        }
      }
      l += sum;
    };
    float x_lo[TT][4], x_hi[TT][4];
    logits_of(0, slope_lo, qinv_lo, x_lo);
    float mn_lo = fmaxf(m_lo, row_max(x_lo)), mn_hi = m_hi;   // finite: the stage's first token is valid
    if (rows16) {
      logits_of(2, slope_hi, qinv_hi, x_hi);
      mn_hi = fmaxf(m_hi, row_max(x_hi));
    }
    // Rescale what earlier stages accumulated only when some row's running maximum moved.
    if (__any_sync(0xffffffffu, mn_lo > m_lo || mn_hi > m_hi)) {
      const float corr_lo = exp2_approx(m_lo - mn_lo);
      l_lo *= corr_lo;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        acc[n][0] *= corr_lo;
        acc[n][1] *= corr_lo;
      }
      if (rows16) {
        const float corr_hi = exp2_approx(m_hi - mn_hi);
        l_hi *= corr_hi;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          acc[n][2] *= corr_hi;
          acc[n][3] *= corr_hi;
        }
      }
      m_lo = mn_lo;
      m_hi = mn_hi;
    }
    probs(x_lo, m_lo, l_lo, pa_lo);
    if (rows16) {
      probs(x_hi, m_hi, l_hi, pa_hi);
    } else {
#pragma unroll
      for (int tt = 0; tt < TT; ++tt) pa_hi[tt][0] = pa_hi[tt][1] = 0u;
    }

    // ---------------- PV
    healthy = __all_sync(0xffffffffu, mbar_wait(bv, par, p.status));
    if (!healthy) break;
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      const int tile_tok0 = stage_tok0 + tt * 16;
      if (TT == 1 || tile_tok0 < t_end) {
        // Cache memory past the context may hold anything (NaNs included): clear those V words.
        const bool partial = tile_tok0 + 16 > t_end;
        const int vt = tile_tok0 + 4 * qi;  // first of this lane's four tokens
        if constexpr (!FP8) {
          uint32_t mk0 = 0xffffffffu, mk1 = 0xffffffffu;
          if (partial) {
            mk0 = (vt < t_end ? 0x0000ffffu : 0u) | (vt + 1 < t_end ? 0xffff0000u : 0u);
            mk1 = (vt + 2 < t_end ? 0x0000ffffu : 0u) | (vt + 3 < t_end ? 0xffff0000u : 0u);
          }
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            uint32_t b0, b1;
            lds64(stage + voff[tt] + n * (8 * BS * 2), b0, b1);
            if (partial) { b0 &= mk0; b1 &= mk1; }
            mma16816<MT>(acc[n], pa_lo[tt][0], pa_hi[tt][0], pa_lo[tt][1], pa_hi[tt][1], b0, b1);
          }
        }
      }
    }
    if constexpr (FP8) {
      // One k32 MMA covers the stage's 32 tokens.  Cache bytes past the context may hold anything (NaN
      // codes included): clear them.  mk[h] masks this lane's four tokens of half h.
      uint32_t mk[2] = {0xffffffffu, 0xffffffffu};
      if (stage_tok0 + 32 > t_end) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int vt = stage_tok0 + h * 16 + 4 * qi;
          mk[h] = (vt < t_end ? 0x000000ffu : 0u) | (vt + 1 < t_end ? 0x0000ff00u : 0u) |
                  (vt + 2 < t_end ? 0x00ff0000u : 0u) | (vt + 3 < t_end ? 0xff000000u : 0u);
        }
      }
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4(stage + voff8 + (n / 2) * (16 * BS), r0, r1, r2, r3);
        r0 &= mk[0]; r1 &= mk[1]; r2 &= mk[0]; r3 &= mk[1];
        mma16832_e4m3(acc[n], pa_lo[0][0], pa_hi[0][0], pa_lo[1][0], pa_hi[1][0], r0, r1);
        mma16832_e4m3(acc[n + 1], pa_lo[0][0], pa_hi[0][0], pa_lo[1][0], pa_hi[1][0], r2, r3);
        mma16832_e4m3(acc[n], pa_lo[0][1], pa_hi[0][1], pa_lo[1][1], pa_hi[1][1], r0, r1);
        mma16832_e4m3(acc[n + 1], pa_lo[0][1], pa_hi[0][1], pa_lo[1][1], pa_hi[1][1], r2, r3);
      }
    }

    // Stage consumed by every lane: hand it back to the copy engine.
    __syncwarp();
    if (i + STAGES < n_mine) issue(i + STAGES);
  }

  // ---- merge the warps' states
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  __syncthreads();  // every warp is done with its ring: the merge buffer may alias it
  float* macc = reinterpret_cast<float*>(smem);                    // [NW][16][ROW_F]
  float* mml = macc + NW * 16 * C::ROW_F;                          // [NW][16][2] = (m, l)
  {
    float* a = macc + (warp * 16 + gi) * C::ROW_F + 2 * qi;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      *reinterpret_cast<float2*>(a + n * 8) = make_float2(acc[n][0], acc[n][1]);
      if (rows16) *reinterpret_cast<float2*>(a + 8 * C::ROW_F + n * 8) = make_float2(acc[n][2], acc[n][3]);
    }
    if (qi == 0) {
      mml[(warp * 16 + gi) * 2 + 0] = m_lo;
      mml[(warp * 16 + gi) * 2 + 1] = l_lo;
      mml[(warp * 16 + gi + 8) * 2 + 0] = m_hi;
      mml[(warp * 16 + gi + 8) * 2 + 1] = l_hi;
    }
  }
  __syncthreads();

  const float vscale = FP8 ? p.v_scale : 1.0f;
  // Combines the four warps' states for (row r, dims d, d + 1): running maximum, denominator, numerators.
  auto cta_reduce = [&](int r, int d, float& M, float& den, float& n0, float& n1) {
    M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, mml[(w * 16 + r) * 2]);
    den = n0 = n1 = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float mw = mml[(w * 16 + r) * 2];
      const float wgt = mw == -INFINITY ? 0.f : exp2_approx(mw - M);  // warps that saw no token weigh nothing
      den += wgt * mml[(w * 16 + r) * 2 + 1];
      const float2 v = *reinterpret_cast<const float2*>(macc + (w * 16 + r) * C::ROW_F + d);
      n0 += wgt * v.x;
      n1 += wgt * v.y;
    }
  };

  if (csize == 1) {
    for (int idx = threadIdx.x; idx < nrows * (HEAD / 2); idx += C::THREADS) {
      const int r = idx / (HEAD / 2), d = (idx % (HEAD / 2)) * 2;
      float M, den, n0, n1;
      cta_reduce(r, d, M, den, n0, n1);
      const float inv = vscale / den;
      const int head = head0 + r;
      if (!partitioned) {
        T* o = reinterpret_cast<T*>(p.out) + (static_cast<int64_t>(seq) * p.num_heads + head) * HEAD + d;
        *reinterpret_cast<uint32_t*>(o) = pack2<T>(n0 * inv, n1 * inv);
      } else {
        const int64_t slot = (static_cast<int64_t>(seq) * p.num_heads + head) * p.max_parts + part;
        T* o = reinterpret_cast<T*>(p.tmp_out) + slot * HEAD + d;
        *reinterpret_cast<uint32_t*>(o) = pack2<T>(n0 * inv, n1 * inv);
        if (d == 0) {
          p.max_logits[slot] = M;   // log2 domain
          p.exp_sums[slot] = den;
        }
      }
    }
    return;
  }

  // ---- cluster mode: every CTA publishes its own (M, den, numerators) in shared memory, then rank 0
  // combines the cluster's results through distributed shared memory and writes the output row.
  cg::cluster_group cluster = cg::this_cluster();
  float* cres = reinterpret_cast<float*>(smem + C::WARP_MERGE_BYTES);  // [16][ROW_F]
  float* cml = cres + 16 * C::ROW_F;                                   // [16][2] = (M, den)
  for (int idx = threadIdx.x; idx < nrows * (HEAD / 2); idx += C::THREADS) {
    const int r = idx / (HEAD / 2), d = (idx % (HEAD / 2)) * 2;
    float M, den, n0, n1;
    cta_reduce(r, d, M, den, n0, n1);
    *reinterpret_cast<float2*>(cres + r * C::ROW_F + d) = make_float2(n0, n1);
    if (d == 0) {
      cml[r * 2] = M;
      cml[r * 2 + 1] = den;
    }
  }
  cluster.sync();
  if (cluster.block_rank() == 0) {
    for (int idx = threadIdx.x; idx < nrows * (HEAD / 2); idx += C::THREADS) {
      const int r = idx / (HEAD / 2), d = (idx % (HEAD / 2)) * 2;
      float M = -INFINITY;
      for (int c = 0; c < csize; ++c) M = fmaxf(M, cluster.map_shared_rank(cml, c)[r * 2]);
      float den = 0.f, n0 = 0.f, n1 = 0.f;
      for (int c = 0; c < csize; ++c) {
        const float* rml = cluster.map_shared_rank(cml, c);
        const float mc = rml[r * 2];
        const float wgt = mc == -INFINITY ? 0.f : exp2_approx(mc - M);
        den += wgt * rml[r * 2 + 1];
        const float2 v = *reinterpret_cast<const float2*>(cluster.map_shared_rank(cres, c) + r * C::ROW_F + d);
        n0 += wgt * v.x;
        n1 += wgt * v.y;
      }
      const float inv = den > 0.f ? vscale / den : 0.f;  // empty context: zeros
      T* o = reinterpret_cast<T*>(p.out) + (static_cast<int64_t>(seq) * p.num_heads + head0 + r) * HEAD + d;
      *reinterpret_cast<uint32_t*>(o) = pack2<T>(n0 * inv, n1 * inv);
    }
  }
  cluster.sync();  // peers keep their shared memory alive until rank 0 has read it
}

// Merge of the partitions' results (the v2 reduce step; reference:
// src/kernels/src/pagedattention.cu:470-566).  grid (num_heads, num_seqs), 128 threads.
// max_logits holds log2-domain maxima, exp_sums the matching sums, tmp_out the
// normalised partial outputs.
template <typename T, int HEAD>
__global__ void __launch_bounds__(128)
paged_decode_merge_kernel(T* __restrict__ out, const float* __restrict__ exp_sums, const float* __restrict__ max_logits,
                          const T* __restrict__ tmp_out, const uint32_t* __restrict__ context_lens, int max_parts,
                          int partition_size) {
  constexpr int NWARP = 4;
  // Launched as a programmatic dependent of the partition kernel: wait until that grid's results are visible.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int head = blockIdx.x, seq = blockIdx.y, num_heads = gridDim.x;
  const int ctx = static_cast<int>(context_lens[seq]);
  const int nparts = (ctx + partition_size - 1) / partition_size;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T* o = out + (static_cast<int64_t>(seq) * num_heads + head) * HEAD;
  const int64_t slot0 = (static_cast<int64_t>(seq) * num_heads + head) * max_parts;
  const T* tp = tmp_out + slot0 * HEAD;
  if (nparts <= 1) {
    for (int d = threadIdx.x; d < HEAD; d += 128) o[d] = nparts == 1 ? tp[d] : from_f32<T>(0.f);
    return;
  }
  extern __shared__ float msm[];        // [max_parts] weights, then [NWARP][HEAD] partial sums
  float* wgt = msm;
  float* part_sum = msm + max_parts;
  __shared__ float red[NWARP];
  __shared__ float red2[NWARP];

  float mx = -INFINITY;
  for (int j = threadIdx.x; j < nparts; j += 128) mx = fmaxf(mx, max_logits[slot0 + j]);
#pragma unroll
  for (int o2 = 16; o2 >= 1; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  float sum = 0.f;
  for (int j = threadIdx.x; j < nparts; j += 128) {
    const float w = exp_sums[slot0 + j] * exp2_approx(max_logits[slot0 + j] - mx);
    wgt[j] = w;
    sum += w;
  }
#pragma unroll
  for (int o2 = 16; o2 >= 1; o2 >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o2);
  if (lane == 0) red2[warp] = sum;
  __syncthreads();
  const float inv = 1.0f / ((red2[0] + red2[1]) + (red2[2] + red2[3]));

  // Each warp sums a strided subset of the partitions; lanes cover the head dimension.
  constexpr int PER_LANE = (HEAD + 31) / 32;
  float a[PER_LANE];
#pragma unroll
  for (int k = 0; k < PER_LANE; ++k) a[k] = 0.f;
  for (int j = warp; j < nparts; j += NWARP) {
    const float w = wgt[j];
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
      const int d = lane + k * 32;
      if (d < HEAD) a[k] += w * to_f32<T>(tp[static_cast<int64_t>(j) * HEAD + d]);
    }
  }
#pragma unroll
  for (int k = 0; k < PER_LANE; ++k) {
    const int d = lane + k * 32;
    if (d < HEAD) part_sum[warp * HEAD + d] = a[k];
  }
  __syncthreads();
  for (int d = threadIdx.x; d < HEAD; d += 128) {
    const float v = (part_sum[d] + part_sum[HEAD + d]) + (part_sum[2 * HEAD + d] + part_sum[3 * HEAD + d]);
    o[d] = from_f32<T>(v * inv);
  }
}

}  // namespace pa
