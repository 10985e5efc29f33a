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
//   * rows land at a pitch of row bytes + 16 in a permuted order of row slots, which makes the
//     two access patterns below free of bank conflicts;
//   * K (both layouts) and V of the flash layout: a lane converts 16 bytes of output of one
//     token - lanes run over tokens first, so a warp's stores fill whole 256-byte runs of a
//     cache page whenever the tokens sit in consecutive slots;
//   * V of the x-layout is a transpose ([token][d] -> [d][token in block]), done by
//     ldmatrix.trans: a lane receives four consecutive tokens of one d as two words, converts
//     them and stores four bytes (eight for a 16-bit cache) when the tokens sit in four aligned
//     consecutive slots - 128-byte (256-byte) runs per warp store when the whole tile does -
//     else element by element (decode steps);
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
// Row slot of token t in a stage (tokens 8..15 swap places in pairs of two: see the V path).
__device__ __forceinline__ int staged_row(int t) { return t ^ ((t >> 2) & 2); }
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

  // a stage: the 16 rows (token t in row slot staged_row(t)), then the 16 slots of the tile
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
      bulk_g2s(smem_u32(st) + staged_row(t) * p.pitch, src, uint32_t(row_bytes), bar, policy);
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
      const unsigned char* rows = st + staged_row(t) * p.pitch;
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
      // ================= V of the x-layout: a transpose ([token][d] -> [d][token in block]), done
      // by ldmatrix.trans.  One instruction hands every lane, for row d = lane / 4 of an 8-d
      // group, two 32-bit words of two tokens each; the token rows that form its 8x8 matrices
      // are chosen so that lane j = lane % 4 receives tokens 4 j .. 4 j + 3 (matrix A = tokens
      // 0 1 4 5 8 9 12 13, matrix B = the others), i.e. four consecutive bytes (fp8) or eight
      // (16-bit cache) of the cache row, in the word format that the quantiser takes.  The row
      // slots (staged_row) make the eight rows of either matrix, and the eight tokens of either
      // half of the tile that the K path reads together, fall into different bank groups.  A lane stores its four tokens with one word store when they sit in four
      // consecutive, aligned slots of one block, else one by one; eight lanes-of-four make a
      // 128-byte (256-byte) run of the cache when the whole tile is such a run.
      const int j = lane & 3;
      // this lane's four tokens: slots, validity, where they go (element index of row d = 0)
      int64_t tb[4];
      bool tv[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t sk = reinterpret_cast<const int64_t*>(st + slot_off)[4 * j + k];
        tv[k] = sk >= 0;
        const int64_t bk = !tv[k] ? 0 : (b_shift >= 0 ? sk >> b_shift : sk / B);
        tb[k] = ((bk * H + h) * int64_t(D) + piece * DP) * B + (tv[k] ? sk - bk * B : 0);
      }
      const int64_t s0 = reinterpret_cast<const int64_t*>(st + slot_off)[4 * j];
      bool quad = tv[0] && tv[1] && tv[2] && tv[3];
#pragma unroll
      for (int k = 1; k < 4; ++k) quad = quad && reinterpret_cast<const int64_t*>(st + slot_off)[4 * j + k] == s0 + k;
      quad = quad && (s0 & 3) == 0 && B % 4 == 0;
      // ldmatrix row address of this lane: matrix lane / 8 = (token set) + 2 * (d half), row lane % 8
      const int mr = lane & 7, mi = lane >> 3;
      const int mtok = (mr >> 1) * 4 + (mr & 1) + (mi & 1) * 2;
      const uint32_t maddr = smem_u32(st) + uint32_t(staged_row(mtok) * p.pitch + (mi >> 1) * 16);
      cache_t* vbase = static_cast<cache_t*>(p.value_cache);
      // One pass over the item's rows.  fp8: the fast pass quantises without looking at the
      // codes and only collects whether any of them is a NaN code (a NaN, or a quotient that
      // overflowed on the way); if so - rare - the item is done again with the division, which
      // overwrites what the fast pass stored.
      auto pass = [&](auto exact_tag) -> uint32_t {
        constexpr bool kExact = decltype(exact_tag)::value;
        (void)kExact;
        uint32_t nan_bits = 0;
        for (int d16 = 0; d16 < DP; d16 += 16) {
          uint32_t r0, r1, r2, r3;  // (tokens 4j, 4j+1), (4j+2, 4j+3) of row d; the same of row d + 8
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                       : "r"(maddr + uint32_t(d16) * 2u));
          const int d = d16 + (lane >> 2);
          uint32_t lo[2], hi[2];  // this lane's piece of row d and of row d + 8 (one word when fp8)
          if constexpr (KV != kKvAuto) {
            if constexpr (kExact) {
              const uint32_t wa[2] = {r0, r1}, wb[2] = {r2, r3};
              uint32_t oa[1], ob[1];
              convert_words<in_t, KV, 2>(wa, oa, v_div);  // (checks its own codes)
              convert_words<in_t, KV, 2>(wb, ob, v_div);
              lo[0] = oa[0];
              hi[0] = ob[0];
            } else {
              const uint32_t va = neg_quant4<in_t, KV == kKvE5M2>(r0, r1, v_div);
              const uint32_t vb = neg_quant4<in_t, KV == kKvE5M2>(r2, r3, v_div);
              nan_bits |= ((va & 0x7F7F7F7Fu) + 0x01010101u) | ((vb & 0x7F7F7F7Fu) + 0x01010101u);
              lo[0] = va ^ 0x80808080u;
              hi[0] = vb ^ 0x80808080u;
            }
            lo[1] = hi[1] = 0;
          } else {
            lo[0] = r0;
            lo[1] = r1;
            hi[0] = r2;
            hi[1] = r3;
          }
          const int64_t rowoff = int64_t(d) * B;  // row d; row d + 8 lies 8 * B elements further
          if (quad) {
            cache_t* dst = vbase + tb[0] + rowoff;
            if constexpr (E == 1) {
              *reinterpret_cast<uint32_t*>(dst) = lo[0];
              *reinterpret_cast<uint32_t*>(dst + 8 * int64_t(B)) = hi[0];
            } else {
              *reinterpret_cast<uint2*>(dst) = make_uint2(lo[0], lo[1]);
              *reinterpret_cast<uint2*>(dst + 8 * int64_t(B)) = make_uint2(hi[0], hi[1]);
            }
          } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (!tv[k]) continue;
              cache_t* dst = vbase + tb[k] + rowoff;
              if constexpr (E == 1) {
                *reinterpret_cast<unsigned char*>(dst) = static_cast<unsigned char>(lo[0] >> (8 * k));
                *reinterpret_cast<unsigned char*>(dst + 8 * int64_t(B)) = static_cast<unsigned char>(hi[0] >> (8 * k));
              } else {
                *reinterpret_cast<uint16_t*>(dst) = static_cast<uint16_t>(lo[k >> 1] >> (16 * (k & 1)));
                *reinterpret_cast<uint16_t*>(dst + 8 * int64_t(B)) = static_cast<uint16_t>(hi[k >> 1] >> (16 * (k & 1)));
              }
            }
          }
        }
        return nan_bits & 0x80808080u;
      };
      if constexpr (KV == kKvAuto) {
        pass(std::false_type{});
      } else {
        // (ldmatrix is warp-collective: the decision to repeat is taken by the warp)
        const bool again = !v_div.fast || __any_sync(0xffffffffu, pass(std::false_type{}) != 0);
        if (again) pass(std::true_type{});
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
