#include "block_pool.hpp"

#include <algorithm>

namespace pa {

BlockPool::BlockPool(int num_blocks, int max_seqs, int max_blocks_per_seq)
    : num_blocks_(num_blocks), max_seqs_(max_seqs), max_blocks_per_seq_(max_blocks_per_seq),
      tables_((size_t)max_seqs * max_blocks_per_seq, -1), len_(max_seqs, 0), nblk_(max_seqs, 0),
      live_(max_seqs, 0), dirty_idx_(max_seqs, -1) {
  free_.resize(num_blocks);
  for (int i = 0; i < num_blocks; i++) free_[i] = num_blocks - 1 - i;  // 0 is handed out first
}

bool BlockPool::set_free_order(const int32_t* order, int n) {
  if (n != num_blocks_ || (int)free_.size() != num_blocks_) return false;
  std::vector<char> seen(num_blocks_, 0);
  for (int i = 0; i < n; i++) {
    if (order[i] < 0 || order[i] >= num_blocks_ || seen[order[i]]) return false;
    seen[order[i]] = 1;
  }
  for (int i = 0; i < n; i++) free_[n - 1 - i] = order[i];
  return true;
}

int BlockPool::create() {
  for (int s = 0; s < max_seqs_; s++)
    if (!live_[s]) {
      live_[s] = 1;
      len_[s] = 0;
      nblk_[s] = 0;
      return s;
    }
  return -1;
}

bool BlockPool::release(int seq) {
  if (!valid(seq)) return false;
  int32_t* t = tables_.data() + (size_t)seq * max_blocks_per_seq_;
  for (int i = nblk_[seq] - 1; i >= 0; i--) {
    free_.push_back(t[i]);
    t[i] = -1;
  }
  live_[seq] = 0;
  len_[seq] = 0;
  nblk_[seq] = 0;
  return true;
}

int BlockPool::reserve(int seq, int new_len) {
  if (!valid(seq) || new_len < 0) return 1;
  if (new_len <= len_[seq]) return 0;
  int want = (new_len + kBlockTokens - 1) / kBlockTokens;
  if (want > max_blocks_per_seq_) return 1;
  int need = want - nblk_[seq];
  if (need > (int)free_.size()) return 2;
  if (need > 0) {
    int32_t* t = tables_.data() + (size_t)seq * max_blocks_per_seq_;
    int lo = nblk_[seq];
    for (int i = 0; i < need; i++) {
      t[lo + i] = free_.back();
      free_.pop_back();
    }
    nblk_[seq] = want;
    int di = dirty_idx_[seq];
    if (di < 0) {
      dirty_idx_[seq] = (int)dirty_.size();
      dirty_.push_back({seq, lo, want});
    } else {
      dirty_[di].lo = std::min(dirty_[di].lo, lo);
      dirty_[di].hi = std::max(dirty_[di].hi, want);
    }
  }
  len_[seq] = new_len;
  return 0;
}

}  // namespace pa
