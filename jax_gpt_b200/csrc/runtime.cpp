// Host-side native runtime: a memory-mapped token-window loader with a prefetch thread and
// pinned staging buffers, and an asynchronous checkpoint writer that streams tensors into
// safetensors files on background threads.
//
// These take the place of the native pieces the reference borrows from its dependencies:
// grain's ArrayRecord / DataLoader workers (jax_gpt/data/pipeline.py:96-128) and Orbax's
// asynchronous TensorStore writer (jax_gpt/trainer/checkpointing.py:28-45).
#include <ATen/ATen.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <torch/library.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <sstream>
#include <set>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

using at::Tensor;

// ------------------------------------------------------------------------------------------
// Token window loader. The file is a flat array of uint16 token ids. Window i covers tokens
// [i*S, i*S + S + 1): inputs are the first S, targets the last S (one token of overlap between
// consecutive windows). A shard sees windows shard_index, shard_index + shard_count, ...
// ------------------------------------------------------------------------------------------
class TokenLoader {
 public:
  TokenLoader(const std::string& path, int64_t seq_len, int64_t micro_batch, int64_t shard_index, int64_t shard_count,
              int64_t prefetch, bool pin)
      : seq_(seq_len), mb_(micro_batch), shard_index_(shard_index), shard_count_(shard_count), pin_(pin) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    TORCH_CHECK(fd_ >= 0, "TokenLoader: cannot open ", path);
    struct stat st;
    TORCH_CHECK(fstat(fd_, &st) == 0, "TokenLoader: fstat failed for ", path);
    n_tokens_ = static_cast<int64_t>(st.st_size) / 2;
    TORCH_CHECK(n_tokens_ > seq_, "TokenLoader: file has fewer than seq_len + 1 tokens");
    map_ = static_cast<const uint16_t*>(mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, fd_, 0));
    TORCH_CHECK(map_ != MAP_FAILED, "TokenLoader: mmap failed");
    map_bytes_ = st.st_size;
    madvise(const_cast<uint16_t*>(map_), map_bytes_, MADV_SEQUENTIAL);
    n_windows_ = (n_tokens_ - 1) / seq_;
    n_local_ = (n_windows_ - shard_index_ + shard_count_ - 1) / shard_count_;
    TORCH_CHECK(n_local_ > 0, "TokenLoader: shard has no windows");
    depth_ = prefetch < 1 ? 1 : prefetch;
    worker_ = std::thread([this] { run(); });
  }

  ~TokenLoader() {
    {
      std::lock_guard<std::mutex> l(mu_);
      stop_ = true;
    }
    cv_space_.notify_all();
    cv_item_.notify_all();
    if (worker_.joinable()) worker_.join();
    if (map_ && map_ != MAP_FAILED) munmap(const_cast<uint16_t*>(map_), map_bytes_);
    if (fd_ >= 0) ::close(fd_);
  }

  std::tuple<Tensor, Tensor> next() {
    std::unique_lock<std::mutex> l(mu_);
    cv_item_.wait(l, [this] { return !queue_.empty() || stop_; });
    TORCH_CHECK(!queue_.empty(), "TokenLoader: stopped");
    auto item = std::move(queue_.front());
    queue_.pop_front();
    l.unlock();
    cv_space_.notify_one();
    return item;
  }

  // Continue from local window `item` (counted within this shard); O(1), no replay.
  void seek(int64_t item) {
    std::unique_lock<std::mutex> l(mu_);
    cursor_ = item;
    ++generation_;
    queue_.clear();
    l.unlock();
    cv_space_.notify_all();
  }

  int64_t num_windows() const { return n_windows_; }
  int64_t num_local_windows() const { return n_local_; }
  int64_t cursor() {
    std::lock_guard<std::mutex> l(mu_);
    return cursor_ - static_cast<int64_t>(queue_.size()) * mb_;
  }

 private:
  void fill(Tensor& x, Tensor& y, int64_t first_item) {
    int32_t* px = x.data_ptr<int32_t>();
    int32_t* py = y.data_ptr<int32_t>();
    for (int64_t b = 0; b < mb_; ++b) {
      const int64_t local = (first_item + b) % n_local_;  // wraps around at the end of the shard (epochs)
      const int64_t w = shard_index_ + local * shard_count_;
      const uint16_t* src = map_ + w * seq_;
      for (int64_t t = 0; t < seq_; ++t) {
        px[b * seq_ + t] = src[t];
        py[b * seq_ + t] = src[t + 1];
      }
    }
  }

  void run() {
    while (true) {
      int64_t item, gen;
      {
        std::unique_lock<std::mutex> l(mu_);
        cv_space_.wait(l, [this] { return stop_ || static_cast<int64_t>(queue_.size()) < depth_; });
        if (stop_) return;
        item = cursor_;
        gen = generation_;
        cursor_ += mb_;
      }
      auto opts = at::TensorOptions().dtype(at::kInt).pinned_memory(pin_);
      Tensor x = at::empty({mb_, seq_}, opts), y = at::empty({mb_, seq_}, opts);
      fill(x, y, item);
      {
        std::lock_guard<std::mutex> l(mu_);
        if (gen == generation_) queue_.emplace_back(std::move(x), std::move(y));  // drop batches made stale by seek()
      }
      cv_item_.notify_one();
    }
  }

  int64_t seq_, mb_, shard_index_, shard_count_;
  bool pin_;
  int fd_ = -1;
  const uint16_t* map_ = nullptr;
  size_t map_bytes_ = 0;
  int64_t n_tokens_ = 0, n_windows_ = 0, n_local_ = 0, depth_ = 1;
  int64_t cursor_ = 0, generation_ = 0;
  bool stop_ = false;
  std::mutex mu_;
  std::condition_variable cv_item_, cv_space_;
  std::deque<std::tuple<Tensor, Tensor>> queue_;
  std::thread worker_;
};

// ------------------------------------------------------------------------------------------
// Asynchronous safetensors writer. A job is a list of (name, CPU tensor) pairs; a worker writes
// "<path>.tmp" (8-byte header length, JSON header, raw tensor bytes) and renames it to <path>.
// Jobs run in submission order on one thread per writer, so a manifest submitted after the
// data files is on disk only when they are.
// ------------------------------------------------------------------------------------------
const char* st_dtype(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return "F32";
    case at::kDouble: return "F64";
    case at::kHalf: return "F16";
    case at::kBFloat16: return "BF16";
    case at::kLong: return "I64";
    case at::kInt: return "I32";
    case at::kShort: return "I16";
    case at::kChar: return "I8";
    case at::kByte: return "U8";
    case at::kBool: return "BOOL";
    case at::kFloat8_e4m3fn: return "F8_E4M3";
    case at::kFloat8_e5m2: return "F8_E5M2";
    default: TORCH_CHECK(false, "AsyncWriter: unsupported dtype for safetensors");
  }
}

struct WriteJob {
  std::string path;
  std::vector<std::string> names;
  std::vector<Tensor> tensors;
  std::string raw;  // when non-empty: write these bytes verbatim (manifests)
};

class AsyncWriter {
 public:
  AsyncWriter() : worker_([this] { run(); }) {}
  ~AsyncWriter() {
    {
      std::lock_guard<std::mutex> l(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    if (worker_.joinable()) worker_.join();
  }
  void submit(WriteJob job) {
    {
      std::lock_guard<std::mutex> l(mu_);
      jobs_.push_back(std::move(job));
      ++pending_;
    }
    cv_.notify_one();
  }
  // Returns false when the wait ran out of time.
  bool wait(double timeout_s) {
    std::unique_lock<std::mutex> l(mu_);
    return cv_done_.wait_for(l, std::chrono::duration<double>(timeout_s), [this] { return pending_ == 0; });
  }
  int64_t pending() {
    std::lock_guard<std::mutex> l(mu_);
    return pending_;
  }
  // Returns the first error since the last call and clears it (later checkpoints start clean).
  std::string last_error() {
    std::lock_guard<std::mutex> l(mu_);
    std::string e;
    e.swap(error_);
    return e;
  }

 private:
  static void write_all(FILE* f, const void* p, size_t n, const std::string& path) {
    TORCH_CHECK(fwrite(p, 1, n, f) == n, "AsyncWriter: short write to ", path);
  }
  // The files of one checkpoint share a directory: once a job of a directory has failed, the later jobs of that
  // directory (above all its manifest, which marks the checkpoint complete) are dropped.
  static std::string dir_of(const std::string& path) {
    const size_t p = path.find_last_of('/');
    return p == std::string::npos ? std::string(".") : path.substr(0, p);
  }
  struct FileCloser {
    FILE* f;
    std::string tmp;
    bool keep = false;
    ~FileCloser() {
      if (f != nullptr) fclose(f);
      if (!keep) remove(tmp.c_str());
    }
  };
  void do_job(const WriteJob& j) {
    const std::string tmp = j.path + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    TORCH_CHECK(f != nullptr, "AsyncWriter: cannot open ", tmp);
    FileCloser guard{f, tmp};   // closes the file and removes the partial ".tmp" if anything below throws
    if (!j.raw.empty()) {
      write_all(f, j.raw.data(), j.raw.size(), tmp);
    } else {
      std::ostringstream h;
      h << "{";
      uint64_t off = 0;
      for (size_t i = 0; i < j.tensors.size(); ++i) {
        const Tensor& t = j.tensors[i];
        const uint64_t nbytes = static_cast<uint64_t>(t.numel()) * t.element_size();
        if (i) h << ",";
        h << "\"" << j.names[i] << "\":{\"dtype\":\"" << st_dtype(t.scalar_type()) << "\",\"shape\":[";
        for (int64_t d = 0; d < t.dim(); ++d) h << (d ? "," : "") << t.size(d);
        h << "],\"data_offsets\":[" << off << "," << off + nbytes << "]}";
        off += nbytes;
      }
      h << "}";
      std::string header = h.str();
      while (header.size() % 8) header.push_back(' ');
      const uint64_t hl = header.size();
      write_all(f, &hl, 8, tmp);
      write_all(f, header.data(), header.size(), tmp);
      for (const Tensor& t : j.tensors)
        write_all(f, t.data_ptr(), static_cast<size_t>(t.numel()) * t.element_size(), tmp);
    }
    TORCH_CHECK(fflush(f) == 0 && fsync(fileno(f)) == 0, "AsyncWriter: flush failed for ", tmp);
    const int rc = fclose(f);
    guard.f = nullptr;
    TORCH_CHECK(rc == 0, "AsyncWriter: close failed for ", tmp);
    TORCH_CHECK(rename(tmp.c_str(), j.path.c_str()) == 0, "AsyncWriter: rename failed for ", j.path);
    guard.keep = true;
  }
  void run() {
    while (true) {
      WriteJob job;
      bool skip = false;
      {
        std::unique_lock<std::mutex> l(mu_);
        cv_.wait(l, [this] { return stop_ || !jobs_.empty(); });
        if (jobs_.empty()) return;
        job = std::move(jobs_.front());
        jobs_.pop_front();
        skip = failed_dirs_.count(dir_of(job.path)) > 0;
      }
      if (!skip) {
        try {
          do_job(job);
        } catch (const std::exception& e) {
          std::lock_guard<std::mutex> l(mu_);
          if (error_.empty()) error_ = e.what();
          failed_dirs_.insert(dir_of(job.path));
        }
      }
      {
        std::lock_guard<std::mutex> l(mu_);
        --pending_;
      }
      cv_done_.notify_all();
    }
  }
  std::mutex mu_;
  std::condition_variable cv_, cv_done_;
  std::deque<WriteJob> jobs_;
  int64_t pending_ = 0;
  bool stop_ = false;
  std::string error_;
  std::set<std::string> failed_dirs_;
  std::thread worker_;
};

// ------------------------------------------------------------------------------------------------
// Block-table manager of the paged KV cache: a free list of pages, the page list and token count of
// every sequence, and host mirrors (pinned when CUDA is present) of the block table and the length
// vector that the cache uploads with one asynchronous copy when they change.
class PageTable {
 public:
  PageTable(int64_t n_pages, int64_t page_size, int64_t max_seqs, int64_t max_pages, bool pin)
      : page_size_(page_size), max_pages_(max_pages), owned_(max_seqs, 0) {
    TORCH_CHECK(n_pages > 0 && page_size > 0 && max_seqs > 0 && max_pages > 0, "page table: bad sizes");
    auto opt = at::TensorOptions().dtype(at::kInt).pinned_memory(pin);
    table_ = at::full({max_seqs, max_pages}, -1, opt);
    lens_ = at::zeros({max_seqs}, opt);
    free_.reserve(n_pages);
    for (int64_t p = n_pages - 1; p >= 0; --p) free_.push_back(static_cast<int32_t>(p));
  }
  // Makes sequence `seq` own enough pages for `new_len` tokens; returns how many pages were added.
  int64_t reserve(int64_t seq, int64_t new_len) {
    std::lock_guard<std::mutex> l(mu_);
    check_seq(seq);
    const int64_t need = (new_len + page_size_ - 1) / page_size_;
    TORCH_CHECK(need <= max_pages_, "paged cache: sequence ", seq, " needs ", need, " pages, the block table has ",
                max_pages_, " columns");
    const int64_t have = owned_[seq];
    if (need <= have) return 0;
    TORCH_CHECK(need - have <= static_cast<int64_t>(free_.size()), "paged cache exhausted: want ", need - have,
                " pages, ", free_.size(), " free");
    int32_t* row = table_.data_ptr<int32_t>() + seq * max_pages_;
    for (int64_t i = have; i < need; ++i) {
      row[i] = free_.back();
      free_.pop_back();
    }
    owned_[seq] = need;
    ++version_;
    return need - have;
  }
  void advance(const std::vector<int64_t>& seqs, int64_t n) {
    std::lock_guard<std::mutex> l(mu_);
    int32_t* lens = lens_.data_ptr<int32_t>();
    for (int64_t s : seqs) {
      check_seq(s);
      TORCH_CHECK((lens[s] + n + page_size_ - 1) / page_size_ <= owned_[s], "paged cache: advance past the reserved pages");
      lens[s] += static_cast<int32_t>(n);
    }
    ++version_;
  }
  void release(int64_t seq) {
    std::lock_guard<std::mutex> l(mu_);
    check_seq(seq);
    int32_t* row = table_.data_ptr<int32_t>() + seq * max_pages_;
    for (int64_t i = owned_[seq] - 1; i >= 0; --i) {
      free_.push_back(row[i]);
      row[i] = -1;
    }
    owned_[seq] = 0;
    lens_.data_ptr<int32_t>()[seq] = 0;
    ++version_;
  }
  int64_t length(int64_t seq) {
    std::lock_guard<std::mutex> l(mu_);
    check_seq(seq);
    return lens_.data_ptr<int32_t>()[seq];
  }
  int64_t n_free() {
    std::lock_guard<std::mutex> l(mu_);
    return static_cast<int64_t>(free_.size());
  }
  int64_t version() {
    std::lock_guard<std::mutex> l(mu_);
    return version_;
  }
  Tensor table() { return table_; }
  Tensor lens() { return lens_; }

 private:
  void check_seq(int64_t s) const { TORCH_CHECK(s >= 0 && s < static_cast<int64_t>(owned_.size()), "paged cache: bad sequence id ", s); }
  int64_t page_size_, max_pages_;
  std::vector<int64_t> owned_;
  std::vector<int32_t> free_;
  Tensor table_, lens_;
  int64_t version_ = 0;
  std::mutex mu_;
};

std::mutex g_mu;
std::unordered_map<int64_t, std::unique_ptr<TokenLoader>> g_loaders;
std::unordered_map<int64_t, std::unique_ptr<AsyncWriter>> g_writers;
std::unordered_map<int64_t, std::unique_ptr<PageTable>> g_tables;
int64_t g_next = 1;

PageTable* page_table(int64_t h) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_tables.find(h);
  TORCH_CHECK(it != g_tables.end(), "unknown page-table handle ", h);
  return it->second.get();
}

TokenLoader* loader(int64_t h) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_loaders.find(h);
  TORCH_CHECK(it != g_loaders.end(), "unknown loader handle ", h);
  return it->second.get();
}
AsyncWriter* writer(int64_t h) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_writers.find(h);
  TORCH_CHECK(it != g_writers.end(), "unknown writer handle ", h);
  return it->second.get();
}

}  // namespace

void b200_register_runtime(torch::Library& m) {
  m.def("loader_create(str path, int seq_len, int micro_batch, int shard_index, int shard_count, int prefetch, bool pin) -> int",
        [](std::string path, int64_t s, int64_t mb, int64_t si, int64_t sc, int64_t pf, bool pin) {
          auto p = std::make_unique<TokenLoader>(path, s, mb, si, sc, pf, pin);
          std::lock_guard<std::mutex> l(g_mu);
          g_loaders[g_next] = std::move(p);
          return g_next++;
        });
  m.def("loader_next(int handle) -> (Tensor, Tensor)", [](int64_t h) { return loader(h)->next(); });
  m.def("loader_seek(int handle, int item) -> ()", [](int64_t h, int64_t item) { loader(h)->seek(item); });
  m.def("loader_num_windows(int handle) -> int", [](int64_t h) { return loader(h)->num_windows(); });
  m.def("loader_num_local_windows(int handle) -> int", [](int64_t h) { return loader(h)->num_local_windows(); });
  m.def("loader_close(int handle) -> ()", [](int64_t h) {
    std::unique_ptr<TokenLoader> p;
    {
      std::lock_guard<std::mutex> l(g_mu);
      auto it = g_loaders.find(h);
      if (it == g_loaders.end()) return;
      p = std::move(it->second);
      g_loaders.erase(it);
    }
  });
  m.def("writer_create() -> int", []() {
    auto p = std::make_unique<AsyncWriter>();
    std::lock_guard<std::mutex> l(g_mu);
    g_writers[g_next] = std::move(p);
    return g_next++;
  });
  m.def("writer_submit_safetensors(int handle, str path, str[] names, Tensor[] tensors) -> ()",
        [](int64_t h, std::string path, std::vector<std::string> names, std::vector<Tensor> tensors) {
          TORCH_CHECK(names.size() == tensors.size(), "writer: names and tensors differ in length");
          for (auto& t : tensors) TORCH_CHECK(t.device().is_cpu() && t.is_contiguous(), "writer: CPU contiguous tensors only");
          writer(h)->submit(WriteJob{std::move(path), std::move(names), std::move(tensors), ""});
        });
  m.def("writer_submit_bytes(int handle, str path, str data) -> ()", [](int64_t h, std::string path, std::string data) {
    if (data.empty()) data = " ";
    writer(h)->submit(WriteJob{std::move(path), {}, {}, std::move(data)});
  });
  m.def("writer_wait(int handle, float timeout_s) -> bool", [](int64_t h, double t) { return writer(h)->wait(t); });
  m.def("writer_pending(int handle) -> int", [](int64_t h) { return writer(h)->pending(); });
  m.def("writer_last_error(int handle) -> str", [](int64_t h) { return writer(h)->last_error(); });
  m.def("pagetable_create(int n_pages, int page_size, int max_seqs, int max_pages, bool pin) -> int",
        [](int64_t n, int64_t ps, int64_t ms, int64_t mp, bool pin) {
          auto p = std::make_unique<PageTable>(n, ps, ms, mp, pin);
          std::lock_guard<std::mutex> l(g_mu);
          g_tables[g_next] = std::move(p);
          return g_next++;
        });
  m.def("pagetable_reserve(int handle, int[] seqs, int[] new_lens) -> int",
        [](int64_t h, std::vector<int64_t> seqs, std::vector<int64_t> lens) {
          TORCH_CHECK(seqs.size() == lens.size(), "pagetable_reserve: one length per sequence");
          int64_t added = 0;
          for (size_t i = 0; i < seqs.size(); ++i) added += page_table(h)->reserve(seqs[i], lens[i]);
          return added;
        });
  m.def("pagetable_advance(int handle, int[] seqs, int n) -> ()",
        [](int64_t h, std::vector<int64_t> seqs, int64_t n) { page_table(h)->advance(seqs, n); });
  m.def("pagetable_release(int handle, int seq) -> ()", [](int64_t h, int64_t s) { page_table(h)->release(s); });
  m.def("pagetable_length(int handle, int seq) -> int", [](int64_t h, int64_t s) { return page_table(h)->length(s); });
  m.def("pagetable_n_free(int handle) -> int", [](int64_t h) { return page_table(h)->n_free(); });
  m.def("pagetable_version(int handle) -> int", [](int64_t h) { return page_table(h)->version(); });
  m.def("pagetable_tensors(int handle) -> (Tensor, Tensor)", [](int64_t h) {
    return std::make_tuple(page_table(h)->table(), page_table(h)->lens());
  });
  m.def("pagetable_close(int handle) -> ()", [](int64_t h) {
    std::lock_guard<std::mutex> l(g_mu);
    g_tables.erase(h);
  });
  m.def("writer_close(int handle) -> ()", [](int64_t h) {
    std::unique_ptr<AsyncWriter> p;
    {
      std::lock_guard<std::mutex> l(g_mu);
      auto it = g_writers.find(h);
      if (it == g_writers.end()) return;
      p = std::move(it->second);
      g_writers.erase(it);
    }
  });
}
