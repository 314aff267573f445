// Host-side runtime pieces that sit on the input and loading paths of a training or serving job:
//
//   * bin packing of documents into fixed-length token streams (first-fit decreasing with a max-tree, or
//     order-preserving greedy) and the collation of packs into the flat arrays the varlen attention kernels read
//     (token ids, boundary-masked labels, per-document positions, cu_seqlens, document start per token), written
//     straight into caller-provided (pinned) buffers by a small thread pool;
//   * parallel positional reads of tensor byte ranges from a checkpoint file into caller-provided buffers
//     (one pread loop per worker, so a multi-gigabyte shard is read with several requests in flight);
//   * a reference-counted block allocator with per-sequence block tables for the paged KV cache
//     (fork shares blocks, append copies a shared tail block on write, truncate and free return blocks).
//
// Everything is plain C++17 with a C ABI; the Python side binds it with ctypes.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

constexpr int64_t kIgnore = -100;

template <class F>
void parallel_for(int64_t n, int threads, F&& fn) {
  if (threads <= 0) threads = static_cast<int>(std::thread::hardware_concurrency());
  threads = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(threads, n)));
  if (threads == 1) {
    for (int64_t i = 0; i < n; ++i) fn(i);
    return;
  }
  std::atomic<int64_t> next{0};
  std::vector<std::thread> pool;
  pool.reserve(threads);
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([&] {
      for (int64_t i = next.fetch_add(1); i < n; i = next.fetch_add(1)) fn(i);
    });
  for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------------------------------------- packing
// First-fit decreasing. lens[i] is clipped to cap by the caller. Documents shorter than min_len get bin -1.
// Ties keep input order; the first bin with room is found through a max-tree over remaining capacities, so the
// result equals a linear first-fit scan. Returns the number of bins.
int64_t pm_pack_ffd(const int32_t* lens, int64_t n, int32_t cap, int32_t min_len, int32_t* bin_of) {
  std::vector<int64_t> order;
  order.reserve(n);
  for (int64_t i = 0; i < n; ++i) {
    bin_of[i] = -1;
    if (lens[i] >= min_len && lens[i] <= cap && lens[i] > 0) order.push_back(i);
  }
  std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return lens[a] > lens[b]; });
  int64_t leaves = 1;
  while (leaves < static_cast<int64_t>(std::max<size_t>(order.size(), 1))) leaves *= 2;
  std::vector<int32_t> tree(2 * leaves, cap);
  int64_t bins = 0;
  for (int64_t idx : order) {
    const int32_t need = lens[idx];
    int64_t node = 1;
    while (node < leaves) node = tree[2 * node] >= need ? 2 * node : 2 * node + 1;
    const int64_t b = node - leaves;
    bin_of[idx] = static_cast<int32_t>(b);
    bins = std::max(bins, b + 1);
    tree[node] -= need;
    for (node /= 2; node; node /= 2) tree[node] = std::max(tree[2 * node], tree[2 * node + 1]);
  }
  return bins;
}

// Order-preserving greedy: a document that does not fit closes the current bin.
int64_t pm_pack_greedy(const int32_t* lens, int64_t n, int32_t cap, int32_t min_len, int32_t* bin_of) {
  int64_t bin = 0;
  int64_t used = 0;
  bool open = false;
  for (int64_t i = 0; i < n; ++i) {
    bin_of[i] = -1;
    if (lens[i] < min_len || lens[i] > cap || lens[i] <= 0) continue;
    if (open && used + lens[i] > cap) {
      ++bin;
      used = 0;
    }
    bin_of[i] = static_cast<int32_t>(bin);
    used += lens[i];
    open = true;
  }
  return open ? bin + 1 : 0;
}

// Collate packs into one token stream.
//   tokens / labels : flat int32 arrays of all documents (labels may be null: the ids are the labels)
//   doc_off[d], doc_len[d] : start of document d in the flat arrays and how many of its tokens are used
//   pack_docs[pack_off[p] .. pack_off[p+1]) : documents of pack p in stream order
//   pack_len > 0 : every pack is right-padded to pack_len by one pseudo-document of ignored pad tokens
// Outputs (sized by the caller: T = sum over packs of max(tokens, pack_len); cu has one entry per document and pad
// document plus one): ids / labels int64, pos / seq_start int32, cu int32.
// meta = {T, n_cu, real tokens, documents, longest document}.
// Labels: the first token of every document after the first in its pack is ignored (the shifted loss would train
// the previous document's last token to predict it), and so is the first token of every pack after the first.
int pm_collate_packs(const int32_t* tokens, const int32_t* labels, const int64_t* doc_off, const int32_t* doc_len,
                     const int64_t* pack_docs, const int64_t* pack_off, int64_t n_packs, int64_t pack_len,
                     int32_t pad_id, int mask_boundaries, int64_t* out_ids, int64_t* out_labels, int32_t* out_pos,
                     int32_t* out_seq_start, int32_t* out_cu, int64_t* meta, int threads) {
  std::vector<int64_t> t0(n_packs + 1, 0), c0(n_packs + 1, 0);
  int64_t real = 0, ndocs = 0, longest = 0;
  for (int64_t p = 0; p < n_packs; ++p) {
    int64_t tok = 0;
    for (int64_t j = pack_off[p]; j < pack_off[p + 1]; ++j) {
      const int64_t n = doc_len[pack_docs[j]];
      tok += n;
      longest = std::max(longest, n);
    }
    if (pack_len > 0 && tok > pack_len) return -1;
    const int64_t nd = pack_off[p + 1] - pack_off[p];
    const bool padded = pack_len > 0 && tok < pack_len;
    real += tok;
    ndocs += nd;
    t0[p + 1] = t0[p] + std::max(tok, pack_len);
    c0[p + 1] = c0[p] + nd + (padded ? 1 : 0);
  }
  out_cu[0] = 0;
  parallel_for(n_packs, threads, [&](int64_t p) {
    int64_t t = t0[p];
    int64_t c = c0[p] + 1;
    for (int64_t j = pack_off[p]; j < pack_off[p + 1]; ++j) {
      const int64_t d = pack_docs[j];
      const int64_t n = doc_len[d];
      const int32_t* src = tokens + doc_off[d];
      const int32_t* lab = labels ? labels + doc_off[d] : src;
      for (int64_t i = 0; i < n; ++i) {
        out_ids[t + i] = src[i];
        out_labels[t + i] = lab[i];
        out_pos[t + i] = static_cast<int32_t>(i);
        out_seq_start[t + i] = static_cast<int32_t>(t);
      }
      if (n > 0 && ((mask_boundaries && j > pack_off[p]) || (j == pack_off[p] && p > 0))) out_labels[t] = kIgnore;
      t += n;
      out_cu[c++] = static_cast<int32_t>(t);
    }
    const int64_t end = t0[p + 1];
    if (t < end) {
      const int64_t start = t;
      for (int64_t i = 0; t < end; ++t, ++i) {
        out_ids[t] = pad_id;
        out_labels[t] = kIgnore;
        out_pos[t] = static_cast<int32_t>(i);
        out_seq_start[t] = static_cast<int32_t>(start);
      }
      out_cu[c++] = static_cast<int32_t>(t);
    }
  });
  meta[0] = t0[n_packs];
  meta[1] = c0[n_packs] + 1;
  meta[2] = real;
  meta[3] = ndocs;
  meta[4] = longest;
  return 0;
}

// ---------------------------------------------------------------------------------------------- checkpoint reads
// Reads n byte ranges [offs[i], offs[i] + sizes[i]) of `path` into dst[i]. Ranges above 64 MiB are split so that
// several workers share one large tensor. Returns 0, or -errno of the first failure (-EIO for a short read).
int pm_read_ranges(const char* path, int64_t n, const int64_t* offs, const int64_t* sizes, void* const* dst,
                   int threads) {
  const int fd = ::open(path, O_RDONLY);
  if (fd < 0) return -errno;
  struct Piece {
    int64_t off, size;
    char* dst;
  };
  constexpr int64_t kChunk = int64_t(64) << 20;
  std::vector<Piece> pieces;
  for (int64_t i = 0; i < n; ++i)
    for (int64_t o = 0; o < sizes[i]; o += kChunk)
      pieces.push_back({offs[i] + o, std::min(kChunk, sizes[i] - o), static_cast<char*>(dst[i]) + o});
  std::atomic<int> err{0};
  parallel_for(static_cast<int64_t>(pieces.size()), threads, [&](int64_t i) {
    if (err.load(std::memory_order_relaxed)) return;
    const Piece& pc = pieces[i];
    int64_t done = 0;
    while (done < pc.size) {
      const ssize_t r = ::pread(fd, pc.dst + done, static_cast<size_t>(pc.size - done), pc.off + done);
      if (r < 0) {
        if (errno == EINTR) continue;
        err.store(-errno);
        return;
      }
      if (r == 0) {
        err.store(-EIO);
        return;
      }
      done += r;
    }
  });
  ::close(fd);
  return err.load();
}

// ---------------------------------------------------------------------------------------------- KV block allocator
struct PmBlockPool {
  int32_t block_size;
  std::vector<int32_t> free_list;     // LIFO: the most recently released block is reused first
  std::vector<int32_t> refs;
  struct Seq {
    std::vector<int32_t> blocks;
    int64_t len = 0;
  };
  std::unordered_map<int64_t, Seq> seqs;
};

void* pm_pool_create(int32_t num_blocks, int32_t block_size) {
  auto* p = new PmBlockPool();
  p->block_size = block_size;
  p->refs.assign(num_blocks, 0);
  p->free_list.resize(num_blocks);
  for (int32_t i = 0; i < num_blocks; ++i) p->free_list[i] = num_blocks - 1 - i;   // block 0 is handed out first
  return p;
}
void pm_pool_destroy(void* h) { delete static_cast<PmBlockPool*>(h); }
int32_t pm_pool_num_free(void* h) { return static_cast<int32_t>(static_cast<PmBlockPool*>(h)->free_list.size()); }
int32_t pm_pool_ref(void* h, int32_t block) { return static_cast<PmBlockPool*>(h)->refs[block]; }

int pm_pool_add(void* h, int64_t seq) {
  auto* p = static_cast<PmBlockPool*>(h);
  if (p->seqs.count(seq)) return -1;
  p->seqs[seq];
  return 0;
}
int64_t pm_pool_length(void* h, int64_t seq) {
  auto* p = static_cast<PmBlockPool*>(h);
  auto it = p->seqs.find(seq);
  return it == p->seqs.end() ? -1 : it->second.len;
}
int32_t pm_pool_num_blocks(void* h, int64_t seq) {
  auto* p = static_cast<PmBlockPool*>(h);
  auto it = p->seqs.find(seq);
  return it == p->seqs.end() ? -1 : static_cast<int32_t>(it->second.blocks.size());
}
static void pool_release(PmBlockPool* p, int32_t b) {
  if (--p->refs[b] == 0) p->free_list.push_back(b);
}
int pm_pool_free(void* h, int64_t seq) {
  auto* p = static_cast<PmBlockPool*>(h);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return -1;
  for (int32_t b : it->second.blocks) pool_release(p, b);
  p->seqs.erase(it);
  return 0;
}
// Blocks that appending n tokens would take from the free list (a shared, partly filled tail block costs one more
// because it is copied before the first write).
int32_t pm_pool_blocks_needed(void* h, int64_t seq, int64_t n) {
  auto* p = static_cast<PmBlockPool*>(h);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return -1;
  const auto& s = it->second;
  const int64_t bs = p->block_size;
  int64_t need = (s.len + n + bs - 1) / bs - static_cast<int64_t>(s.blocks.size());
  if (n > 0 && s.len % bs != 0 && !s.blocks.empty() && p->refs[s.blocks.back()] > 1) ++need;
  return static_cast<int32_t>(std::max<int64_t>(need, 0));
}
// Reserve room for n more tokens. slots[n] receives the flat cache slot of every new token
// (block * block_size + offset). When the tail block is shared it is replaced by a fresh block and
// copy_src/copy_dst (one entry each) name the block copy the caller must perform first; *n_copies is 0 or 1.
// Returns 0, -1 for an unknown sequence, -2 when the pool has too few free blocks (nothing is changed then).
int pm_pool_reserve(void* h, int64_t seq, int64_t n, int64_t* slots, int32_t* copy_src, int32_t* copy_dst,
                    int32_t* n_copies) {
  auto* p = static_cast<PmBlockPool*>(h);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return -1;
  *n_copies = 0;
  if (pm_pool_blocks_needed(h, seq, n) > static_cast<int32_t>(p->free_list.size())) return -2;
  auto& s = it->second;
  const int64_t bs = p->block_size;
  if (n > 0 && s.len % bs != 0 && p->refs[s.blocks.back()] > 1) {
    const int32_t fresh = p->free_list.back();
    p->free_list.pop_back();
    p->refs[fresh] = 1;
    copy_src[0] = s.blocks.back();
    copy_dst[0] = fresh;
    *n_copies = 1;
    pool_release(p, s.blocks.back());
    s.blocks.back() = fresh;
  }
  for (int64_t i = 0; i < n; ++i) {
    const int64_t pos = s.len + i;
    if (pos / bs >= static_cast<int64_t>(s.blocks.size())) {
      const int32_t b = p->free_list.back();
      p->free_list.pop_back();
      p->refs[b] = 1;
      s.blocks.push_back(b);
    }
    slots[i] = static_cast<int64_t>(s.blocks[pos / bs]) * bs + pos % bs;
  }
  s.len += n;
  return 0;
}
int pm_pool_truncate(void* h, int64_t seq, int64_t new_len) {
  auto* p = static_cast<PmBlockPool*>(h);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end() || new_len < 0 || new_len > it->second.len) return -1;
  auto& s = it->second;
  const int64_t keep = (new_len + p->block_size - 1) / p->block_size;
  for (size_t i = static_cast<size_t>(keep); i < s.blocks.size(); ++i) pool_release(p, s.blocks[i]);
  if (static_cast<int64_t>(s.blocks.size()) > keep) s.blocks.resize(static_cast<size_t>(keep));
  s.len = new_len;
  return 0;
}
// dst becomes a copy of src that shares every block (reference counts go up; no data moves).
int pm_pool_fork(void* h, int64_t src, int64_t dst) {
  auto* p = static_cast<PmBlockPool*>(h);
  auto it = p->seqs.find(src);
  if (it == p->seqs.end() || p->seqs.count(dst)) return -1;
  PmBlockPool::Seq copy = it->second;
  for (int32_t b : copy.blocks) ++p->refs[b];
  p->seqs[dst] = std::move(copy);
  return 0;
}
// Fill a [n_seqs, max_blocks] table (padded with 0) and seq_lens for a decode or prefill launch.
int pm_pool_tables(void* h, const int64_t* seq_ids, int64_t n_seqs, int32_t max_blocks, int32_t* table,
                   int32_t* seq_lens) {
  auto* p = static_cast<PmBlockPool*>(h);
  for (int64_t i = 0; i < n_seqs; ++i) {
    auto it = p->seqs.find(seq_ids[i]);
    if (it == p->seqs.end()) return -1;
    const auto& s = it->second;
    if (static_cast<int32_t>(s.blocks.size()) > max_blocks) return -2;
    int32_t* row = table + i * max_blocks;
    std::copy(s.blocks.begin(), s.blocks.end(), row);
    std::fill(row + s.blocks.size(), row + max_blocks, 0);
    seq_lens[i] = static_cast<int32_t>(s.len);
  }
  return 0;
}

}  // extern "C"
