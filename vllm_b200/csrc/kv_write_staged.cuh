// Staged KV write: the main path of reshape_and_cache / reshape_and_cache_flash for 16-bit
// key/value tensors (csrc/cache_kernels.cu:225-358 of the reference).
//
// The write is a gather of token rows, a per-element conversion and a scatter into cache pages.
// With plain loads every thread waits for its loads, converts and stores, and nothing else is
// in flight meanwhile; measured on B200 that reached about half of the copy bandwidth.  Here the
// loads are decoupled from the arithmetic:
//   * one persistent CTA per SM; every WARP is an independent worker with a private ring of
//     shared-memory stages and mbarriers (no CTA-wide barrier at all);
//   * a work item is 16 consecutive tokens of one head of K, or of V: its 16 rows (head_size
//     elements each) are fetched with one bulk async copy per row, issued by 16 lanes at once,
//     up to `stages - 1` items ahead of the one being converted;
//   * rows land at a pitch of row bytes + 16, which makes the two access patterns below free of
//     bank conflicts;
//   * K (both layouts) and V of the flash layout: a lane converts 16 bytes of output of one
//     token - lanes run over tokens first, so a warp's stores fill whole 256-byte runs of a
//     cache page whenever the tokens sit in consecutive slots;
//   * V of the x-layout is a transpose ([token][d] -> [d][token in block]): a lane reads two
//     adjacent d of all 16 tokens from shared memory, converts the two rows and writes each
//     with one 16-byte store when the tile fills 16 aligned consecutive slots, else four bytes
//     at a time where consecutive tokens allow it, else element by element (decode steps);
//   * small writes cut a head of 128 into two work items (hsplit), which halves the latency of
//     the one item a warp then has;
//   * the kShift instantiation (large x-layout writes) moves a tile whose tokens are consecutive
//     positions of a sequence onto the next 16-slot boundary of the cache, so that prefill
//     chunks which start inside a block still write whole rows of V (details at `shift_of`);
//   * every mbarrier wait is bounded; a wait that runs out records a status code and the warp
//     leaves.
#pragma once

#include "decode_common.cuh"

namespace b200pa {

struct StagedWriteParams {
  const void* key;
  const void* value;
  void* key_cache;
  void* value_cache;
  const int64_t* slot_mapping;
  const float* k_scale;
  const float* v_scale;
  int* status;
  int64_t key_stride;    // elements
  int64_t value_stride;
  int64_t block_stride;  // flash layout: elements of the cache
  int64_t page_stride;
  int64_t head_stride;
  int num_tokens;
  int num_heads;
  int head_size;
  int block_size;
  int nstages;
  int pitch;        // bytes between two token rows of a stage
  int stage_bytes;  // 16 rows + slot table (+ shifts)
  int hsplit;       // pieces a head's row is cut into (1 or 2): each piece is a work item
};

constexpr int kStagedTile = 16;  // tokens per work item
constexpr int kStagedMaxWarps = 24;

// 16 input elements (two 16-byte shared-memory reads) -> 16 bytes of cache, or 8 -> 16 for a
// 16-bit cache (plain copy).
template <typename in_t, typename cache_t, int KV>
__device__ __forceinline__ uint4 staged_chunk(const unsigned char* src, const ScaledDiv& div) {
  if constexpr (KV == kKvAuto) {
    return *reinterpret_cast<const uint4*>(src);
  } else {
    const uint4 a = reinterpret_cast<const uint4*>(src)[0];
    const uint4 b = reinterpret_cast<const uint4*>(src)[1];
    const uint32_t wi[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t wo[4];
    convert_words<in_t, KV, 8>(wi, wo, div);
    return make_uint4(wo[0], wo[1], wo[2], wo[3]);
  }
}

template <typename in_t, typename cache_t, int KV, bool kFlash, bool kShift>
__global__ void __launch_bounds__(kStagedMaxWarps * 32, 1) kv_write_staged_kernel(const StagedWriteParams p) {
  static_assert(!(kFlash && kShift), "tiles are moved in the x-layout only");
  static_assert(sizeof(in_t) == 2, "16-bit key/value tensors");
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int E = sizeof(cache_t);       // 1 (fp8) or 2
  constexpr int CH = 16 / E;               // elements per 16-byte chunk of cache (= x)
  constexpr int CHB = CH * 2;              // bytes of input that feed one chunk
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int D = p.head_size;
  const int H = p.num_heads;
  const int B = p.block_size;
  const int NST = p.nstages;
  const int HS = p.hsplit;
  const int DP = D / HS;  // head dimensions of one work item
  const int row_bytes = DP * 2;
  const int b_shift = (B & (B - 1)) == 0 ? 31 - __clz(B) : -1;
  const int tiles = (p.num_tokens + kStagedTile - 1) / kStagedTile;
  // Items: the (tile, head) pairs of K, then those of V, dealt out SM-first.  Every warp walks
  // through both halves, so the K and V work (which differ in cost in the x-layout) is spread
  // evenly over warps and SMs.
  const unsigned HH = unsigned(H) * unsigned(HS);  // (head, piece of the head) pairs per tile
  const unsigned pairs = unsigned(tiles) * HH;
  // pair number / HH by one multiply-high (exact while pairs * HH < 2^32): the item bookkeeping
  // would otherwise spend four runtime divisions per item
  const uint32_t hh_m = HH > 1 ? 0xFFFFFFFFu / HH + 1 : 0;  // ceil(2^32 / HH)
  const bool hh_fast = uint64_t(pairs) * HH <= 0xFFFFFFFFull;
  auto div_hh = [&](unsigned n) -> unsigned { return HH == 1 ? n : (hh_fast ? __umulhi(n, hh_m) : n / HH); };
  const unsigned items = pairs * 2u;
  const unsigned grid_warps = gridDim.x * unsigned(nwarps);
  unsigned next_item = unsigned(warp) * gridDim.x + blockIdx.x;

  // ---- shared memory: [mbarriers of all warps][stages of warp 0][stages of warp 1]...
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
  const uint32_t bars_bytes = (uint32_t(nwarps) * NST * 8 + 127u) & ~127u;
  unsigned char* my_stages = smem_raw + bars_bytes + size_t(warp) * NST * p.stage_bytes;
  const uint32_t my_bar0 = smem_u32(bars) + uint32_t(warp) * NST * 8;
  if (lane == 0) {
    for (int s = 0; s < NST; ++s) mbar_init(my_bar0 + s * 8, 1);
    fence_barrier_init();
  }
  __syncwarp();

  const char* key_b = static_cast<const char*>(p.key);
  const char* val_b = static_cast<const char*>(p.value);
  const uint64_t policy = policy_evict_first();

  // a stage: 16 rows, then the 16 slots of the tile
  const int slot_off = kStagedTile * p.pitch;

  // The slot of a token is needed before its row can be requested; it is loaded two items ahead
  // (`slot_a` belongs to the item that the next produce() call will request, `slot_b` to the one
  // after), so that the producer never waits for that load.  The load is a volatile asm
  // statement: the compiler would otherwise move it down to its use.
  // kShift: lanes 16, 17 and 18 fetch the first, last and ninth slot of the tile in front as well.
  auto load_slot = [&](unsigned item) -> int64_t {
    if (item >= items) return -1;
    const int tile = int(div_hh(item >= pairs ? item - pairs : item));
    int tok = tile * kStagedTile + (lane & 15);
    if constexpr (kShift) {
      if (lane >= 16)
        tok = lane < 19 ? (tile - 1) * kStagedTile + (lane == 16 ? 0 : (lane == 17 ? kStagedTile - 1 : 8)) : -1;
    }
    if (tok < 0 || tok >= p.num_tokens) return -1;
    int64_t v;
    asm volatile("ld.global.nc.s64 %0, [%1];" : "=l"(v) : "l"(p.slot_mapping + tok));
    return v;
  };
  // ---- kShift: which 16 tokens an item covers.  A row of V in the x-layout holds the tokens
  // of one block, so a tile writes whole 16-byte rows only if its tokens fill 16 aligned slots;
  // the tiles of a prefill chunk that starts inside a block never do.  A tile whose first,
  // ninth and last token sit at consecutive offsets modulo 16 (consecutive positions of one
  // sequence, whatever blocks they are in) therefore covers the 16 tokens from the next 16-slot
  // boundary on: tokens [16 i + shift, 16 i + shift + 16), 0 <= shift < 16.  The tokens
  // [16 i, 16 i + shift) that it gives up lie in the window of tile i - 1 if that one is shifted
  // by at least as much - every tile can tell, the shift is a function of a tile's own slots
  // (three of them, and the same function for a tile and for its successor looking back at it);
  // otherwise tile i writes them itself from global memory (`head` in the consumer; once per
  // run).  Windows may overlap: a slot is then written twice with the same bytes.  The rule is
  // only a guess about the slots; whatever they are, every token is written, with its own slot.
  auto shift_of = [&](int64_t first, int64_t mid, int64_t last) -> int {
    if (first < 0 || mid < 0 || last < 0) return 0;
    if (((mid - first) & 15) != 8 || ((last - first) & 15) != 15) return 0;
    return int((kStagedTile - (first & 15)) & 15);
  };
  // Turns the slots of a tile (as load_slot delivers them) into those of its window; `sh` =
  // shift | shift of the tile in front << 8.
  auto to_window = [&](unsigned item, int64_t cand, int& sh) -> int64_t {
    sh = 0;
    if constexpr (!kShift) {
      return cand;
    } else {
      if (item >= items) return cand;
      const int64_t f = __shfl_sync(0xffffffffu, cand, 0), m = __shfl_sync(0xffffffffu, cand, 8);
      const int64_t l = __shfl_sync(0xffffffffu, cand, 15);
      const int64_t pf = __shfl_sync(0xffffffffu, cand, 16), pl = __shfl_sync(0xffffffffu, cand, 17);
      const int64_t pm = __shfl_sync(0xffffffffu, cand, 18);
      const int d = shift_of(f, m, l);
      if (d == 0) return cand;  // (the shift of the tile in front does not matter then)
      // the tile in front, by the very rule that its own warp applies
      const int dp = shift_of(pf, pm, pl);
      sh = d | (dp << 8);
      const int tile = int(div_hh(item >= pairs ? item - pairs : item));
      const int tok = tile * kStagedTile + d + (lane & 15);
      if (tok >= p.num_tokens) return -1;
      int64_t v;
      asm volatile("ld.global.nc.s64 %0, [%1];" : "=l"(v) : "l"(p.slot_mapping + tok));
      return v;
    }
  };
  int sh_a = 0;
  int64_t slot_a = to_window(next_item, load_slot(next_item), sh_a);
  int64_t slot_b = load_slot(next_item + grid_warps);

  // a stage: 16 rows, the 16 slots of the tile (window), then the shifts
  const int sh_off = slot_off + kStagedTile * 8;

  auto produce = [&](unsigned item, int stage) {
    const bool is_v = item >= pairs;
    const unsigned pr = is_v ? item - pairs : item;
    const int tile = int(div_hh(pr));
    const int hp = int(pr - unsigned(tile) * HH);  // head * HS + piece
    const int t = lane & 15;
    const int sh = sh_a;
    const int tok = tile * kStagedTile + (sh & 0xff) + t;
    const int64_t slot = slot_a;
    // b becomes a (its slots have had an item's time to arrive; a moved window's slots are
    // requested now and have another)
    slot_a = to_window(item + grid_warps, slot_b, sh_a);
    slot_b = load_slot(item + 2 * grid_warps);
    unsigned char* st = my_stages + size_t(stage) * p.stage_bytes;
    if (lane < kStagedTile) reinterpret_cast<int64_t*>(st + slot_off)[t] = slot;
    if constexpr (kShift) {
      if (lane == 0) *reinterpret_cast<int*>(st + sh_off) = sh;
    }
    const bool valid = slot >= 0 && lane < kStagedTile;
    const unsigned vmask = __ballot_sync(0xffffffffu, valid);
    const uint32_t bar = my_bar0 + stage * 8;
    if (lane == 0) mbar_expect_tx(bar, uint32_t(__popc(vmask)) * uint32_t(row_bytes));
    __syncwarp();  // the expectation is set before any copy can complete on the barrier
    if (valid) {
      const char* src = (is_v ? val_b : key_b) +
                        (int64_t(tok) * (is_v ? p.value_stride : p.key_stride) + int64_t(hp) * DP) * 2;
      bulk_g2s(smem_u32(st) + t * p.pitch, src, uint32_t(row_bytes), bar, policy);
    }
  };

  // ---- fill the ring
  int prod_stage = 0, cons_stage = 0, inflight = 0;
  uint32_t cons_phase = 0;
  unsigned cur_item = next_item;
  while (inflight < NST && next_item < items) {
    produce(next_item, prod_stage);
    next_item += grid_warps;
    prod_stage = prod_stage + 1 == NST ? 0 : prod_stage + 1;
    ++inflight;
  }

  // (the scales are read after the first rows have been requested: their latency hides behind
  // the copies)
  const ScaledDiv k_div(KV == kKvAuto ? 1.f : *p.k_scale);
  const ScaledDiv v_div(KV == kKvAuto ? 1.f : *p.v_scale);

  while (inflight > 0) {
    if (!__all_sync(0xffffffffu, mbar_wait(my_bar0 + cons_stage * 8, cons_phase))) {
      if (lane == 0) atomicExch(p.status, kStatusMbarTimeout);
      // give the copies still in flight a bounded chance to land before the shared memory goes
      for (int i = 1; i < inflight; ++i) {
        cons_stage = cons_stage + 1 == NST ? 0 : cons_stage + 1;
        if (cons_stage == 0) cons_phase ^= 1;
        mbar_wait(my_bar0 + cons_stage * 8, cons_phase);
      }
      return;
    }
    const unsigned char* st = my_stages + size_t(cons_stage) * p.stage_bytes;
    const bool is_v = cur_item >= pairs;
    const unsigned cur_pr = is_v ? cur_item - pairs : cur_item;
    const int cur_tile = int(div_hh(cur_pr));
    const int hp = int(cur_pr - unsigned(cur_tile) * HH);
    const int h = HS == 2 ? hp >> 1 : hp;
    const int piece = hp - h * HS;
    // lane t (and t + 16) knows token t's cache block and offset
    const int64_t slot = reinterpret_cast<const int64_t*>(st + slot_off)[lane & 15];
    const bool valid = slot >= 0;
    // (block sizes are powers of two in practice; a 64-bit division per item otherwise)
    const int64_t blk = !valid ? 0 : (b_shift >= 0 ? slot >> b_shift : slot / B);
    const int off = valid ? int(slot - blk * B) : 0;
    const unsigned vmask = __ballot_sync(0xffffffffu, valid) & 0xffffu;

    if constexpr (kShift) {
      // ---- tokens in front of a moved window that no other window covers (see above): at most
      // 15, straight from global memory, all loads independent of each other
      const int sh = *reinterpret_cast<const int*>(st + sh_off);
      const int tile = cur_tile;
      const int hb = tile * kStagedTile + (tile > 0 ? ((sh >> 8) & 0xff) : 0);
      const int nh = min(tile * kStagedTile + (sh & 0xff), p.num_tokens) - hb;
      if (nh > 0) {
        const int64_t hslot = lane < nh ? p.slot_mapping[hb + lane] : int64_t(-1);
        const int64_t in_stride = is_v ? p.value_stride : p.key_stride;
        const unsigned char* rows0 = reinterpret_cast<const unsigned char*>(is_v ? val_b : key_b) +
                                     (int64_t(hb) * in_stride + int64_t(hp) * DP) * 2;
        if (!is_v) {
          const int chunks = D / CH, my_chunks = DP / CH;
          const int total = nh * my_chunks;
          for (int base = 0; base < total; base += 32) {  // (uniform trip count: shuffles inside)
            const int idx = base + lane;
            const bool act = idx < total;
            const int k = act ? idx / my_chunks : 0;
            const int c = idx - k * my_chunks;
            const int64_t hs = __shfl_sync(0xffffffffu, hslot, k);
            if (act && hs >= 0) {
              const int64_t hblk = b_shift >= 0 ? hs >> b_shift : hs / B;
              const int hoff = int(hs - hblk * B);
              unsigned char* dst = static_cast<unsigned char*>(p.key_cache) +
                                   (((hblk * H + h) * int64_t(chunks) + piece * my_chunks + c) * B + hoff) * 16;
              *reinterpret_cast<uint4*>(dst) =
                  staged_chunk<in_t, cache_t, KV>(rows0 + int64_t(k) * in_stride * 2 + c * CHB, k_div);
            }
          }
        } else {
          const int quads = DP / 4;  // a lane converts four adjacent d of one token at a time
          const int total = nh * quads;
          for (int base = 0; base < total; base += 32) {
            const int idx = base + lane;
            const bool act = idx < total;
            const int k = act ? idx / quads : 0;
            const int q4 = idx - k * quads;
            const int64_t hs = __shfl_sync(0xffffffffu, hslot, k);
            if (act && hs >= 0) {
              const int64_t hblk = b_shift >= 0 ? hs >> b_shift : hs / B;
              const int hoff = int(hs - hblk * B);
              const uint2 raw = __ldg(reinterpret_cast<const uint2*>(rows0 + int64_t(k) * in_stride * 2) + q4);
              in_t four[4];
              *reinterpret_cast<uint2*>(four) = raw;
              cache_t o[4];
              convert_n<in_t, cache_t, KV, 4>(four, o, v_div);
              cache_t* dst = static_cast<cache_t*>(p.value_cache) +
                             ((hblk * H + h) * int64_t(D) + piece * DP + 4 * q4) * B + hoff;
#pragma unroll
              for (int i = 0; i < 4; ++i) dst[int64_t(i) * B] = o[i];
            }
          }
        }
      }
    }

    if (kFlash || !is_v) {
      // ================= K (and V of the flash layout): 16-byte chunks, tokens first
      const int chunks = D / CH;       // of the whole head
      const int my_chunks = DP / CH;   // of this item
      const int c_first = piece * my_chunks;
      const int t = lane & 15;
      const ScaledDiv& div = is_v ? v_div : k_div;
      const unsigned char* rows = st + t * p.pitch;
      unsigned char* dst;
      int64_t cstep;  // bytes between two chunks of one token in the cache
      if constexpr (kFlash) {
        dst = static_cast<unsigned char*>(is_v ? p.value_cache : p.key_cache) +
              (blk * p.block_stride + int64_t(off) * p.page_stride + int64_t(h) * p.head_stride) * E;
        cstep = 16;
      } else {
        dst = static_cast<unsigned char*>(p.key_cache) +
              (((blk * H + h) * int64_t(chunks)) * B + off) * 16;
        cstep = int64_t(B) * 16;
      }
      if (valid) {
        for (int c = lane >> 4; c < my_chunks; c += 2) {
          const uint4 v = staged_chunk<in_t, cache_t, KV>(rows + c * CHB, div);
          *reinterpret_cast<uint4*>(dst + (c_first + c) * cstep) = v;
        }
      }
    } else {
      // ================= V of the x-layout: transpose, two adjacent d per lane
      const int64_t s0 = __shfl_sync(0xffffffffu, slot, 0);
      const bool in_run = (lane >= kStagedTile) || slot == s0 + lane;
      const bool full_run = __all_sync(0xffffffffu, in_run) && vmask == 0xffffu && s0 % kStagedTile == 0 &&
                            B % kStagedTile == 0;
      constexpr int W4 = 4 / E;  // tokens per 4-byte store
      // tokens that start a 4-byte group: aligned slot, the next W4 - 1 tokens follow in the block
      bool follows = valid;
#pragma unroll
      for (int k = 1; k < W4; ++k) {
        const int64_t sk = __shfl_down_sync(0xffffffffu, slot, k);
        follows &= ((lane & 15) + k < kStagedTile) && sk == slot + k;
      }
      const unsigned starts =
          __ballot_sync(0xffffffffu, follows && (off * E) % 4 == 0 && off + W4 <= B && (B * E) % 4 == 0) & 0xffffu;
      unsigned char* vbase = static_cast<unsigned char*>(p.value_cache);
      const unsigned char* vrows = st;
      // every lane runs every iteration (the stores below use warp shuffles); lanes whose pair
      // of rows lies beyond the head size only take part in those
      const int d_first = piece * DP;
      for (int d_base = 0; d_base < DP; d_base += 64) {
        const int dl = d_base + 2 * lane;  // inside the item
        const int d0 = d_first + dl;       // inside the head
        const bool mine = dl < DP;
        uint32_t two[kStagedTile];  // token t: (d0, d0 + 1)
        if (mine) {
          const unsigned char* col = vrows + dl * 2;
          const int pitch = p.pitch;
#pragma unroll
          for (int t = 0; t < kStagedTile; ++t) two[t] = *reinterpret_cast<const uint32_t*>(col + t * pitch);
        } else {
#pragma unroll
          for (int t = 0; t < kStagedTile; ++t) two[t] = 0u;
        }
        if (vmask != 0xffffu) {  // stale shared memory in the rows of skipped tokens
#pragma unroll
          for (int t = 0; t < kStagedTile; ++t)
            if (!((vmask >> t) & 1u)) two[t] = 0u;
        }
        __align__(16) cache_t c0[kStagedTile], c1[kStagedTile];
        if constexpr (KV != kKvAuto) {
          // row d0 takes the low halves of consecutive tokens' words, row d0 + 1 the high halves
          uint32_t w0[kStagedTile / 2], w1[kStagedTile / 2], o0[kStagedTile / 4], o1[kStagedTile / 4];
#pragma unroll
          for (int t = 0; t < kStagedTile; t += 2) {
            w0[t / 2] = __byte_perm(two[t], two[t + 1], 0x5410u);
            w1[t / 2] = __byte_perm(two[t], two[t + 1], 0x7632u);
          }
          convert_words<in_t, KV, kStagedTile / 2>(w0, o0, v_div);
          convert_words<in_t, KV, kStagedTile / 2>(w1, o1, v_div);
#pragma unroll
          for (int i = 0; i < kStagedTile / 4; ++i) {
            reinterpret_cast<uint32_t*>(c0)[i] = o0[i];
            reinterpret_cast<uint32_t*>(c1)[i] = o1[i];
          }
        } else {
#pragma unroll
          for (int t = 0; t < kStagedTile; t += 2) {
            reinterpret_cast<uint32_t*>(c0)[t / 2] = __byte_perm(two[t], two[t + 1], 0x5410u);
            reinterpret_cast<uint32_t*>(c1)[t / 2] = __byte_perm(two[t], two[t + 1], 0x7632u);
          }
        }
        if (full_run) {
          const int64_t b0 = b_shift >= 0 ? s0 >> b_shift : s0 / B;
          unsigned char* dst = vbase + (((b0 * H + h) * int64_t(D) + d0) * B + int(s0 - b0 * B)) * E;
          if (mine) {
#pragma unroll
            for (int w = 0; w < kStagedTile * E / 16; ++w) {
              reinterpret_cast<uint4*>(dst)[w] = reinterpret_cast<const uint4*>(c0)[w];
              reinterpret_cast<uint4*>(dst + int64_t(B) * E)[w] = reinterpret_cast<const uint4*>(c1)[w];
            }
          }
        } else {
          unsigned covered = 0;  // tokens written as part of an earlier group
#pragma unroll
          for (int t = 0; t < kStagedTile; ++t) {
            if (!((vmask >> t) & 1u) || ((covered >> t) & 1u)) continue;  // warp-uniform
            const int64_t bt = __shfl_sync(0xffffffffu, blk, t);
            const int ot = __shfl_sync(0xffffffffu, off, t);
            unsigned char* dst = vbase + (((bt * H + h) * int64_t(D) + d0) * B + ot) * E;
            if (!mine) continue;
            if (W4 > 1 && ((starts >> t) & 1u) && t + W4 <= kStagedTile) {
              __align__(4) cache_t g0[W4], g1[W4];
#pragma unroll
              for (int k = 0; k < W4; ++k) {
                g0[k] = c0[(t + k) % kStagedTile];
                g1[k] = c1[(t + k) % kStagedTile];
              }
              *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(g0);
              *reinterpret_cast<uint32_t*>(dst + int64_t(B) * E) = *reinterpret_cast<const uint32_t*>(g1);
              covered |= ((1u << W4) - 1u) << t;
            } else {
              *reinterpret_cast<cache_t*>(dst) = c0[t];
              *reinterpret_cast<cache_t*>(dst + int64_t(B) * E) = c1[t];
            }
          }
        }
      }
    }

    // ---- release the stage and refill it
    __syncwarp();
    cons_stage = cons_stage + 1 == NST ? 0 : cons_stage + 1;
    if (cons_stage == 0) cons_phase ^= 1;
    --inflight;
    cur_item += grid_warps;
    if (next_item < items) {
      produce(next_item, prod_stage);
      next_item += grid_warps;
      prod_stage = prod_stage + 1 == NST ? 0 : prod_stage + 1;
      ++inflight;
    }
  }
}

}  // namespace b200pa
