// Host side of the paged KV cache: free list, per-sequence block tables and the
// record of which table entries still have to reach the device mirror.
//
// The reference keeps one contiguous [8, max_seq_len, 64] tensor per layer
// (src/runtime/attention.hpp:47-54) and its paged-attention header is empty
// (src/pagedattention/paged_attention.hpp), so the semantics here are this
// library's own; they are kept deterministic so that a seeded run reproduces
// its tables exactly:
//   * free blocks are handed out LIFO; the initial order is 0,1,2,... unless
//     set_free_order() installs another permutation;
//   * freeing a sequence returns its blocks in reverse table order, so the
//     block freed last is the next one handed out;
//   * reserve() is all-or-nothing and never shrinks;
//   * create() returns the lowest unused sequence id.
#pragma once
#include <cstdint>
#include <vector>

namespace pa {

constexpr int kBlockTokens = 16;

class BlockPool {
 public:
  BlockPool(int num_blocks, int max_seqs, int max_blocks_per_seq);

  int num_blocks() const { return num_blocks_; }
  int max_seqs() const { return max_seqs_; }
  int max_blocks_per_seq() const { return max_blocks_per_seq_; }
  int free_blocks() const { return (int)free_.size(); }

  bool set_free_order(const int32_t* order, int n);  // false unless all blocks are free and order is a permutation
  int create();                                       // -1 when all ids are in use
  bool release(int seq);
  // 0 ok, 1 bad argument (unknown seq, negative length, table too small), 2 out of blocks
  int reserve(int seq, int new_len);
  bool valid(int seq) const { return seq >= 0 && seq < max_seqs_ && live_[seq]; }
  int length(int seq) const { return len_[seq]; }
  int table_size(int seq) const { return nblk_[seq]; }
  const int32_t* table(int seq) const { return tables_.data() + (size_t)seq * max_blocks_per_seq_; }
  const int32_t* all_tables() const { return tables_.data(); }

  // Table entries [lo, hi) of `seq` changed since the last clear_dirty().
  struct Dirty { int seq, lo, hi; };
  const std::vector<Dirty>& dirty() const { return dirty_; }
  void clear_dirty() { dirty_.clear(); dirty_idx_.assign(max_seqs_, -1); }

 private:
  int num_blocks_, max_seqs_, max_blocks_per_seq_;
  std::vector<int32_t> free_;    // back() is handed out next
  std::vector<int32_t> tables_;  // [max_seqs][max_blocks_per_seq]
  std::vector<int> len_, nblk_;
  std::vector<char> live_;
  std::vector<Dirty> dirty_;
  std::vector<int> dirty_idx_;   // seq -> index in dirty_, -1 if clean
};

}  // namespace pa
