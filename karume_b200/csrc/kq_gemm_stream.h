// How the streamed prefill GEMM (kq_qgemm_i4.cu, pair form) deals work to the SM pairs: plain
// integer arithmetic shared by the kernel, its launcher and a host-side test.
//
// The work is `tiles` pair tiles of `ksteps` k-steps each, numbered as units
// tile * ksteps + k-step.  Pair p of `pairs` takes the contiguous run of units
// [p * U / pairs, (p + 1) * U / pairs), U = tiles * ksteps, and cuts it at the tile boundaries
// into fragments.  The fragment that holds a tile's first k-step owns the tile: it adds the sums
// of the pairs after it that hold the tile's other k-steps ("pieces"), in pair order, and
// stores.  A pair has at most one piece, and it is its first fragment.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define KQ_HD __host__ __device__ __forceinline__
#else
#define KQ_HD inline
#endif

namespace kq {
namespace stream {

enum Kind : uint32_t {
  kFinal = 0,  // a whole tile: bias added, stored
  kSlice = 1,  // (not streamed) one K slice of a tile, summed by the reduce kernel
  kPiece = 2,  // k-steps of a tile that starts in an earlier pair: sums left in the pair's slot
  kOwner = 3   // the first k-steps of a tile that continues in later pairs: adds their pieces
};

struct Fragment {
  uint32_t tile;           // pair tile
  uint32_t ks_begin;       // first k-step of the fragment inside the tile
  uint32_t ksteps;         // k-steps of the fragment
  uint32_t kind;           // Kind
  uint32_t tile_end_unit;  // the unit after the tile's last
};

// first unit of pair `pair` (pair == pairs gives the total)
KQ_HD uint32_t run_begin(uint32_t pair, uint64_t units, uint32_t pairs) {
  return static_cast<uint32_t>(pair * units / pairs);
}

// how many fragments the run [begin, end) has
KQ_HD uint32_t fragment_count(uint32_t begin, uint32_t end, uint32_t ksteps) {
  return end > begin ? (end - 1) / ksteps - begin / ksteps + 1 : 0;
}

// the f-th fragment of the run [begin, end)
KQ_HD Fragment fragment(uint32_t begin, uint32_t end, uint32_t ksteps, uint32_t f) {
  Fragment r;
  r.tile = begin / ksteps + f;
  const uint32_t tile_unit = r.tile * ksteps;
  const uint32_t lo = begin > tile_unit ? begin : tile_unit;
  const uint32_t hi = end < tile_unit + ksteps ? end : tile_unit + ksteps;
  r.ks_begin = lo - tile_unit;
  r.ksteps = hi - lo;
  r.tile_end_unit = tile_unit + ksteps;
  r.kind = r.ks_begin != 0 ? kPiece : (r.ksteps < ksteps ? kOwner : kFinal);
  return r;
}

// how many pairs after `pair` hold k-steps of the tile that ends at tile_end_unit
KQ_HD uint32_t partners(uint32_t pair, uint32_t tile_end_unit, uint64_t units, uint32_t pairs) {
  uint32_t n = 0;
  while (pair + n + 1 < pairs && run_begin(pair + n + 1, units, pairs) < tile_end_unit) ++n;
  return n;
}

// Whether a launch is streamed: more than one wave of pair tiles, the last wave of whole tiles
// would leave 15 % or more of the machine's time unused, and a run is at least one tile long
// (a tile then has at most two holders).  A pure function of the shapes.
inline bool worth_streaming(uint32_t tiles, uint32_t pairs, uint32_t ksteps) {
  if (pairs < 2 || tiles <= pairs) return false;
  const uint32_t waves = (tiles + pairs - 1) / pairs;
  const uint64_t units = static_cast<uint64_t>(tiles) * ksteps;
  return static_cast<uint64_t>(tiles) * 100 <= static_cast<uint64_t>(waves) * pairs * 85 && units / pairs >= ksteps &&
         units < (1ull << 31);
}

}  // namespace stream
}  // namespace kq
