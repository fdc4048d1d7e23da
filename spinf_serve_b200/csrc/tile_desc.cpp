// Host-side tile descriptor of the tree mask: which 128x128 (query block, key block) tiles of a packed stream the attention
// kernel must visit, and which of them need no mask evaluation. Same classification as the reference's block tables
// (spinf_serve/packer.py:426-491), restated over per-block summaries:
//   skip     j > i; or (sliding) every real query position of block i is at least `window` past every real key position of j;
//            or the blocks share no job; or every key subtree of block j ends at or before block i's first row
//   full     j < i, both blocks lie inside one job and hold no pad, every key's subtree covers all of block i (not for sliding)
//   partial  everything else that is visited (the diagonal always is)
// flags: bit 0 = full (the reference's classification), bit 1 = the kernel may skip the mask evaluation (equal to bit 0 on the
// full-attention table; on the sliding table also set for tree-full tiles that lie wholly inside the window).
// Streams with images (grp[t] = the image a placeholder token belongs to, -1 elsewhere; an image's placeholders attend to each
// other both ways): a sliding-table tile is not skipped for the window when its two blocks share an image, and a query block also
// visits the LATER key blocks of its images (partial tiles, after the diagonal).
// The visited blocks of a query block are emitted in ascending order; that order is the kernel's reduction order.
#include <algorithm>
#include <climits>
#include <vector>

#include "../../include/spinf_b200.h"

namespace {
struct BlockInfo {
  std::vector<int32_t> arts;  // distinct job slots of the block's real tokens, ascending
  std::vector<int32_t> imgs;  // distinct images of the block's tokens, ascending
  bool has_pad = false;
  int32_t min_end = INT_MAX, max_end = INT_MIN;    // over all 128 tokens (pads carry -1)
  int64_t min_pos = LLONG_MAX, max_pos = LLONG_MIN;  // over real tokens only
};

bool intersect(const std::vector<int32_t>& a, const std::vector<int32_t>& b) {
  size_t i = 0, j = 0;
  while (i < a.size() && j < b.size()) {
    if (a[i] == b[j]) return true;
    if (a[i] < b[j]) ++i; else ++j;
  }
  return false;
}
bool share_job(const BlockInfo& a, const BlockInfo& b) { return intersect(a.arts, b.arts); }

void sort_unique(std::vector<int32_t>& v) {
  std::sort(v.begin(), v.end());
  v.erase(std::unique(v.begin(), v.end()), v.end());
}
}  // namespace

extern "C" int64_t spinf_tile_desc_build_host_img(const int32_t* art, const int32_t* end, const int32_t* pos, const int32_t* grp, int64_t n,
                                                  int32_t window, int32_t* counts, int32_t* blocks, uint8_t* flags) {
  if (!art || !end || !pos || !counts || !blocks || !flags || n < 0 || n % SPINF_BLOCK != 0) return SPINF_ERR_BAD_ARGUMENT;
  const int64_t nb = n / SPINF_BLOCK;
  std::vector<BlockInfo> info(nb);
  for (int64_t b = 0; b < nb; ++b) {
    BlockInfo& bi = info[b];
    for (int64_t t = b * SPINF_BLOCK; t < (b + 1) * SPINF_BLOCK; ++t) {
      bi.min_end = std::min(bi.min_end, end[t]);
      bi.max_end = std::max(bi.max_end, end[t]);
      if (grp && grp[t] >= 0) bi.imgs.push_back(grp[t]);
      if (art[t] < 0) {
        bi.has_pad = true;
        continue;
      }
      bi.arts.push_back(art[t]);
      bi.min_pos = std::min<int64_t>(bi.min_pos, pos[t]);
      bi.max_pos = std::max<int64_t>(bi.max_pos, pos[t]);
    }
    sort_unique(bi.arts);
    sort_unique(bi.imgs);
  }
  const bool windowed = window > 0;
  int64_t total = 0;
  for (int64_t i = 0; i < nb; ++i) {
    const BlockInfo& qi = info[i];
    const bool one_i = qi.arts.size() == 1 && !qi.has_pad;
    int32_t cnt = 0;
    for (int64_t j = 0; j <= i; ++j) {
      const BlockInfo& kj = info[j];
      bool visit = false, full = false, no_mask = false;
      if (j == i) {
        visit = true;
      } else {
        const bool both_real = !qi.arts.empty() && !kj.arts.empty();
        const bool out_of_window = windowed && both_real && qi.min_pos - kj.max_pos >= window && !intersect(qi.imgs, kj.imgs);
        if (!out_of_window && both_real) {
          const bool one_j = kj.arts.size() == 1 && !kj.has_pad;
          const bool tree_full = one_i && one_j && qi.arts[0] == kj.arts[0] && kj.min_end >= (i + 1) * SPINF_BLOCK;
          if (!windowed && tree_full) {
            visit = full = no_mask = true;
          } else if (share_job(qi, kj) && kj.max_end > i * SPINF_BLOCK) {
            visit = true;
            // sliding table: the tile stays "partial" for the reference's table format, but when every pair attends under
            // the tree rule and every pair lies inside the window the kernel need not evaluate the mask
            no_mask = windowed && tree_full && qi.max_pos - kj.min_pos < window;
          }
        }
      }
      if (visit) {
        blocks[i * nb + cnt] = static_cast<int32_t>(j);
        flags[i * nb + cnt] = static_cast<uint8_t>((full ? 1 : 0) | (no_mask ? 2 : 0));
        ++cnt;
      }
    }
    if (!qi.imgs.empty())  // the later key blocks of this block's images
      for (int64_t j = i + 1; j < nb; ++j)
        if (intersect(qi.imgs, info[j].imgs)) {
          blocks[i * nb + cnt] = static_cast<int32_t>(j);
          flags[i * nb + cnt] = 0;
          ++cnt;
        }
    counts[i] = cnt;
    total += cnt;
  }
  return total;
}

extern "C" int64_t spinf_tile_desc_build_host(const int32_t* art, const int32_t* end, const int32_t* pos, int64_t n, int32_t window,
                                              int32_t* counts, int32_t* blocks, uint8_t* flags) {
  return spinf_tile_desc_build_host_img(art, end, pos, nullptr, n, window, counts, blocks, flags);
}
