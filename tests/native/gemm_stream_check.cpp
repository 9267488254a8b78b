// Host-side check of the streamed GEMM's work partition (karume_b200/csrc/kq_gemm_stream.h):
// for many (tiles, k-steps, pairs) every (tile, k-step) unit is covered exactly once, the
// fragments of a run are in order, a tile has exactly one owner (the fragment with its first
// k-step), the owner's partner count is exactly the number of later pairs that hold k-steps
// of the tile, every such pair holds them as a piece and as its FIRST fragment, and the
// streaming rule only ever picks shapes in which a tile has at most two holders.
// Prints "ok <cases>" or the first violation; exit status 0 / 1.
#include <cstdio>
#include <vector>

#include "kq_gemm_stream.h"

using namespace kq::stream;

static int fail(const char* what, unsigned tiles, unsigned ksteps, unsigned pairs, unsigned a, unsigned b) {
  std::printf("FAIL %s: tiles=%u ksteps=%u pairs=%u (%u, %u)\n", what, tiles, ksteps, pairs, a, b);
  return 1;
}

static int check(unsigned tiles, unsigned ksteps, unsigned pairs) {
  const uint64_t units = static_cast<uint64_t>(tiles) * ksteps;
  std::vector<int> covered(units, 0);
  std::vector<int> owner(tiles, -1), holders(tiles, 0);
  std::vector<unsigned> owner_partners(tiles, 0);
  if (run_begin(0, units, pairs) != 0 || run_begin(pairs, units, pairs) != units) return fail("run ends", tiles, ksteps, pairs, 0, 0);
  for (unsigned p = 0; p < pairs; ++p) {
    const unsigned begin = run_begin(p, units, pairs), end = run_begin(p + 1, units, pairs);
    if (end < begin) return fail("run order", tiles, ksteps, pairs, p, 0);
    const unsigned count = fragment_count(begin, end, ksteps);
    unsigned at = begin;
    for (unsigned f = 0; f < count; ++f) {
      const Fragment fr = fragment(begin, end, ksteps, f);
      if (fr.ksteps == 0 || fr.tile >= tiles) return fail("empty or stray fragment", tiles, ksteps, pairs, p, f);
      if (fr.tile * ksteps + fr.ks_begin != at) return fail("fragments not contiguous", tiles, ksteps, pairs, p, f);
      if (fr.tile_end_unit != (fr.tile + 1) * ksteps) return fail("tile end", tiles, ksteps, pairs, p, f);
      for (unsigned i = 0; i < fr.ksteps; ++i) covered[at + i]++;
      at += fr.ksteps;
      holders[fr.tile]++;
      const bool first_kstep = fr.ks_begin == 0, whole = fr.ksteps == ksteps;
      const unsigned want = !first_kstep ? kPiece : (whole ? kFinal : kOwner);
      if (fr.kind != want) return fail("kind", tiles, ksteps, pairs, p, f);
      if (fr.kind == kPiece && f != 0) return fail("a piece that is not the pair's first fragment", tiles, ksteps, pairs, p, f);
      if (first_kstep) {
        if (owner[fr.tile] != -1) return fail("two owners", tiles, ksteps, pairs, p, fr.tile);
        owner[fr.tile] = static_cast<int>(p);
        owner_partners[fr.tile] = fr.kind == kOwner ? partners(p, fr.tile_end_unit, units, pairs) : 0;
      } else if (owner[fr.tile] < 0 || owner[fr.tile] >= static_cast<int>(p)) {
        return fail("a piece before its owner", tiles, ksteps, pairs, p, fr.tile);
      }
    }
    if (at != end) return fail("run not exhausted", tiles, ksteps, pairs, p, at);
  }
  for (uint64_t u = 0; u < units; ++u)
    if (covered[u] != 1) return fail("unit covered != once", tiles, ksteps, pairs, static_cast<unsigned>(u), covered[u]);
  for (unsigned t = 0; t < tiles; ++t) {
    if (owner[t] < 0) return fail("tile without owner", tiles, ksteps, pairs, t, 0);
    if (static_cast<int>(owner_partners[t]) != holders[t] - 1) return fail("partner count", tiles, ksteps, pairs, t, owner_partners[t]);
    if (worth_streaming(tiles, pairs, ksteps) && holders[t] > 2) return fail("streamed tile with three holders", tiles, ksteps, pairs, t, holders[t]);
  }
  return 0;
}

int main() {
  unsigned cases = 0;
  const unsigned tile_counts[] = {1, 2, 3, 16, 56, 64, 73, 74, 75, 112, 148, 149, 224, 225, 448, 896, 1000};
  const unsigned kstep_counts[] = {1, 2, 3, 7, 8, 16, 64, 224};
  const unsigned pair_counts[] = {1, 2, 3, 37, 64, 66, 74};
  for (unsigned tiles : tile_counts)
    for (unsigned ksteps : kstep_counts)
      for (unsigned pairs : pair_counts) {
        if (static_cast<uint64_t>(tiles) * ksteps < pairs) continue;  // the launcher never makes more pairs than units
        if (check(tiles, ksteps, pairs)) return 1;
        ++cases;
      }
  // the rule on the shapes it was measured on (74 resident pairs)
  if (!worth_streaming(224, 74, 64)) return fail("rule: 2048 x 14336, k 4096 must stream", 224, 64, 74, 0, 0);
  if (worth_streaming(896, 74, 64)) return fail("rule: 8192 rows must not stream", 896, 64, 74, 0, 0);
  if (worth_streaming(64, 74, 224)) return fail("rule: one wave must not stream", 64, 224, 74, 0, 0);
  if (worth_streaming(56, 74, 64)) return fail("rule: one wave must not stream", 56, 64, 74, 0, 0);
  std::printf("ok %u\n", cases);
  return 0;
}
