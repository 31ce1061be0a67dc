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
//  * FP8 cache: bytes are widened to f16 with cvt.e4m3x2 on the way into the MMA
//    and the query is converted to f16 once; scales are applied to the fp32 logits
//    and to the fp32 output.
#pragma once

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
  float scale, softcap, k_scale, v_scale;
};

template <typename T, bool FP8, int HEAD, int BS>
struct DecodeCfg {
  using MT = std::conditional_t<FP8, __half, T>;  // MMA input type
  static constexpr int ES = FP8 ? 1 : 2;
  static constexpr int SB = BS >= 16 ? 1 : 16 / BS;  // physical blocks per stage
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
  static constexpr int MERGE_BYTES = NW * 16 * ROW_F * 4 + NW * 16 * 2 * 4;
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
  constexpr int KSTEPS = HEAD / 16;  // MMA k-steps of QK^T
  constexpr int NT = HEAD / 8;       // n-tiles of PV

  const int seq = blockIdx.y;
  const int ctx = static_cast<int>(p.context_lens[seq]);
  const int part = blockIdx.z;
  const int gsplit = (p.group + 15) / 16;               // head sub-groups per kv head (1 unless group > 16)
  const int kvh = blockIdx.x / gsplit;
  const int head0 = kvh * p.group + (blockIdx.x % gsplit) * 16;
  const int nrows = min(16, kvh * p.group + p.group - head0);  // live rows of the M tile
  const bool rows16 = nrows > 8;
  const bool partitioned = p.partition_size > 0;

  int t_begin = 0, t_end = ctx;
  if (partitioned) {
    t_begin = part * p.partition_size;
    if (t_begin >= ctx) return;  // nothing to do for this partition
    t_end = min(ctx, t_begin + p.partition_size);
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gi = lane >> 2, qi = lane & 3;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const uint32_t ring = smem_addr(smem) + warp * (STAGES * STAGE_BYTES);
  const uint32_t bars = smem_addr(smem) + C::DATA_BYTES + warp * (STAGES * 16);  // [stage]{K,V}

  if (ctx == 0) {
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

  // ---- this warp's share of the range: stages warp, warp + NW, ...
  const int n_stages_cta = (t_end - t_begin + STOK - 1) / STOK;
  const int n_mine = n_stages_cta > warp ? (n_stages_cta - warp + NW - 1) / NW : 0;
  const int last_block = (ctx - 1) / BS;  // last physical-block slot of the sequence that holds tokens
  const uint32_t* table = p.block_tables + static_cast<int64_t>(seq) * p.max_num_blocks_per_seq;
  const int64_t head_off = static_cast<int64_t>(kvh) * p.kv_head_stride;
  const unsigned char* kc = reinterpret_cast<const unsigned char*>(p.k_cache);
  const unsigned char* vc = reinterpret_cast<const unsigned char*>(p.v_cache);
  const uint64_t policy = policy_evict_first();

  // Block-table entries for a window of 32 of this warp's stages live one per lane.
  // blk(i, b) = table slot of block b of local stage i.
  auto slot_of = [&](int i, int b) { return (t_begin / BS) + (warp + i * NW) * SB + b; };
  auto load_entries = [&](int round, uint32_t (&e)[SB]) {
    const int i = round * 32 + lane;
#pragma unroll
    for (int b = 0; b < SB; ++b) {
      const int slot = slot_of(i, b);
      e[b] = (i < n_mine && slot <= last_block) ? table[slot] : 0xffffffffu;
    }
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
  uint32_t qa[KSTEPS][4];
  {
    const T* qbase = reinterpret_cast<const T*>(p.q) + static_cast<int64_t>(seq) * p.q_stride + static_cast<int64_t>(head0) * HEAD;
    auto ldq = [&](int row, int col) -> uint32_t {  // two consecutive elements as MT pair
      if (row >= nrows) return 0u;
      const uint32_t raw = *reinterpret_cast<const uint32_t*>(qbase + row * HEAD + col);
      if constexpr (std::is_same<T, MT>::value) {
        return raw;
      } else {  // bf16 query, f16 MMA (FP8 cache)
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 f = __bfloat1622float2(v);
        return pack2<__half>(f.x, f.y);
      }
    };
#pragma unroll
    for (int j = 0; j < KSTEPS; ++j) {
      if constexpr (!FP8) {
        qa[j][0] = ldq(gi, 16 * j + 2 * qi);
        qa[j][1] = ldq(gi + 8, 16 * j + 2 * qi);
        qa[j][2] = ldq(gi, 16 * j + 8 + 2 * qi);
        qa[j][3] = ldq(gi + 8, 16 * j + 8 + 2 * qi);
      } else {  // k-slot permutation matching the byte order of the FP8 chunks
        qa[j][0] = ldq(gi, 16 * j + 4 * qi);
        qa[j][1] = ldq(gi + 8, 16 * j + 4 * qi);
        qa[j][2] = ldq(gi, 16 * j + 4 * qi + 2);
        qa[j][3] = ldq(gi + 8, 16 * j + 4 * qi + 2);
      }
    }
  }

  // ---- per-lane shared-memory offsets
  // K (ldmatrix row addresses).  Matrix mi = lane / 8, row r = lane % 8.
  uint32_t koff[TT];
  {
    const int mi = lane >> 3, r = lane & 7;
    const int tile = FP8 ? (mi & 1) : (mi >> 1);     // which n-tile this matrix feeds
    const int chunk = FP8 ? (mi >> 1) : (mi & 1);    // which 16-byte chunk of the k-step (pair)
    const int tau = 4 * (r >> 1) + (r & 1) + ((((r >> 2) ^ tile) & 1) ? 2 : 0);
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      const int ts = tt * 16 + tau;
      koff[tt] = (ts / BS) * TILE_BYTES + (chunk * BS + (ts % BS)) * 16;
    }
  }
  // V.  16-bit: one 8-byte load per n-tile at row gi; FP8: ldmatrix rows.
  uint32_t voff[TT];
#pragma unroll
  for (int tt = 0; tt < TT; ++tt) {
    if constexpr (FP8) {
      const int mi = lane >> 3, r = lane & 7;
      voff[tt] = SB * TILE_BYTES + (mi * 8 + r) * BS + tt * 16;
    } else if constexpr (BS >= 16) {
      voff[tt] = SB * TILE_BYTES + (gi * BS + tt * 16 + 4 * qi) * 2;
    } else {
      voff[tt] = SB * TILE_BYTES + (qi >> 1) * TILE_BYTES + (gi * BS + (qi & 1) * 4) * 2;
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

  for (int i = 0; i < n_mine && healthy; ++i) {
    const int s = i % STAGES;
    const uint32_t par = (i / STAGES) & 1;
    const uint32_t stage = ring + s * STAGE_BYTES;
    const uint32_t bk = bars + s * 16, bv = bk + 8;
    const int stage_tok0 = t_begin + (warp + i * NW) * STOK;

    // Rotate the block-table window when the stage to be issued this iteration enters a new round.
    if (((i + STAGES) >> 5) > ent_round + 1) {
#pragma unroll
      for (int b = 0; b < SB; ++b) ent_cur[b] = ent_nxt[b];
      ++ent_round;
      load_entries(ent_round + 1, ent_nxt);
    }

    healthy = __all_sync(0xffffffffu, mbar_wait(bk, par, p.status));
    if (!healthy) break;

    // ---------------- logits of up to TT tiles
    float sc[TT][2][4];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
#pragma unroll
      for (int h = 0; h < 2; ++h) sc[tt][h][0] = sc[tt][h][1] = sc[tt][h][2] = sc[tt][h][3] = 0.f;
      if (stage_tok0 + tt * 16 < t_end) {
        if constexpr (!FP8) {
#pragma unroll
          for (int j = 0; j < KSTEPS; ++j) {
            uint32_t r0, r1, r2, r3;
            ldmatrix_x4(stage + koff[tt] + j * (2 * BS * 16), r0, r1, r2, r3);
            mma16816<MT>(sc[tt][0], qa[j][0], qa[j][1], qa[j][2], qa[j][3], r0, r1);
            mma16816<MT>(sc[tt][1], qa[j][0], qa[j][1], qa[j][2], qa[j][3], r2, r3);
          }
        } else {
#pragma unroll
          for (int j = 0; j < KSTEPS; j += 2) {
            uint32_t r0, r1, r2, r3;
            ldmatrix_x4(stage + koff[tt] + (j / 2) * (2 * BS * 16), r0, r1, r2, r3);
            mma16816<MT>(sc[tt][0], qa[j][0], qa[j][1], qa[j][2], qa[j][3], e4m3x2_to_f16x2(r0), e4m3x2_to_f16x2(r0 >> 16));
            mma16816<MT>(sc[tt][1], qa[j][0], qa[j][1], qa[j][2], qa[j][3], e4m3x2_to_f16x2(r1), e4m3x2_to_f16x2(r1 >> 16));
            mma16816<MT>(sc[tt][0], qa[j + 1][0], qa[j + 1][1], qa[j + 1][2], qa[j + 1][3], e4m3x2_to_f16x2(r2), e4m3x2_to_f16x2(r2 >> 16));
            mma16816<MT>(sc[tt][1], qa[j + 1][0], qa[j + 1][1], qa[j + 1][2], qa[j + 1][3], e4m3x2_to_f16x2(r3), e4m3x2_to_f16x2(r3 >> 16));
          }
        }
      }
    }

    // ---------------- online softmax, per tile
    uint32_t pa_lo[TT][2], pa_hi[TT][2];  // P fragments: [tile][k-lo / k-hi]
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      const int tile_tok0 = stage_tok0 + tt * 16;
      pa_lo[tt][0] = pa_lo[tt][1] = pa_hi[tt][0] = pa_hi[tt][1] = 0u;
      if (tile_tok0 < t_end) {
        const int ta = tile_tok0 + tokA, tb = tile_tok0 + tokB;
        const bool v0 = ta < t_end, v1 = ta + 1 < t_end, v2 = tb < t_end, v3 = tb + 1 < t_end;
        auto row = [&](float x0, float x1, float x2, float x3, float slope, float& m, float& l, float& corr,
                       uint32_t& pA, uint32_t& pB) {
          if (plain) {
            x0 *= qk_scale_log2; x1 *= qk_scale_log2; x2 *= qk_scale_log2; x3 *= qk_scale_log2;
          } else {
            x0 *= qk_scale; x1 *= qk_scale; x2 *= qk_scale; x3 *= qk_scale;
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
          x0 = v0 ? x0 : -INFINITY; x1 = v1 ? x1 : -INFINITY; x2 = v2 ? x2 : -INFINITY; x3 = v3 ? x3 : -INFINITY;
          float mx = fmaxf(fmaxf(x0, x1), fmaxf(x2, x3));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          const float mn = fmaxf(m, mx);   // finite: token tile_tok0 is valid
          corr = exp2_approx(m - mn);
          const float p0 = exp2_approx(x0 - mn), p1 = exp2_approx(x1 - mn);
          const float p2 = exp2_approx(x2 - mn), p3 = exp2_approx(x3 - mn);
          l = l * corr + ((p0 + p1) + (p2 + p3));
          m = mn;
          pA = pack2<MT>(p0, p1);
          pB = pack2<MT>(p2, p3);
        };
        float corr_lo, corr_hi = 1.f;
        uint32_t pA, pB;
        row(sc[tt][0][0], sc[tt][0][1], sc[tt][1][0], sc[tt][1][1], slope_lo, m_lo, l_lo, corr_lo, pA, pB);
        // lane q pairs (tokens 4q,4q+1) with V's low word and (4q+2,4q+3) with its high word
        pa_lo[tt][0] = (qi & 2) ? pB : pA;
        pa_lo[tt][1] = (qi & 2) ? pA : pB;
        if (rows16) {
          row(sc[tt][0][2], sc[tt][0][3], sc[tt][1][2], sc[tt][1][3], slope_hi, m_hi, l_hi, corr_hi, pA, pB);
          pa_hi[tt][0] = (qi & 2) ? pB : pA;
          pa_hi[tt][1] = (qi & 2) ? pA : pB;
        }
        // Rescale what earlier tiles accumulated to the new running maximum.
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          acc[n][0] *= corr_lo;
          acc[n][1] *= corr_lo;
        }
        if (rows16) {
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            acc[n][2] *= corr_hi;
            acc[n][3] *= corr_hi;
          }
        }

        // ---------------- PV of this tile
        if (tt == 0) {
          healthy = __all_sync(0xffffffffu, mbar_wait(bv, par, p.status));
        }
        if (healthy) {
          // Validity masks for V words of a partial tile (cache memory past the context may hold NaNs).
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
          } else {
            uint32_t mk = 0xffffffffu;
            if (partial) {
              mk = (vt < t_end ? 0x000000ffu : 0u) | (vt + 1 < t_end ? 0x0000ff00u : 0u) |
                   (vt + 2 < t_end ? 0x00ff0000u : 0u) | (vt + 3 < t_end ? 0xff000000u : 0u);
            }
#pragma unroll
            for (int n = 0; n < NT; n += 4) {
              uint32_t r[4];
              ldmatrix_x4(stage + voff[tt] + (n / 4) * (32 * BS), r[0], r[1], r[2], r[3]);
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const uint32_t w = r[u] & mk;
                mma16816<MT>(acc[n + u], pa_lo[tt][0], pa_hi[tt][0], pa_lo[tt][1], pa_hi[tt][1], e4m3x2_to_f16x2(w),
                             e4m3x2_to_f16x2(w >> 16));
              }
            }
          }
        }
      }
    }
    if (!healthy) break;

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
  for (int idx = threadIdx.x; idx < nrows * (HEAD / 2); idx += C::THREADS) {
    const int r = idx / (HEAD / 2), d = (idx % (HEAD / 2)) * 2;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, mml[(w * 16 + r) * 2]);
    float den = 0.f, n0 = 0.f, n1 = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float wgt = exp2_approx(mml[(w * 16 + r) * 2] - M);  // 0 for warps that saw no token
      den += wgt * mml[(w * 16 + r) * 2 + 1];
      const float2 v = *reinterpret_cast<const float2*>(macc + (w * 16 + r) * C::ROW_F + d);
      n0 += wgt * v.x;
      n1 += wgt * v.y;
    }
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
