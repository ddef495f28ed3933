// Memory-mapped reader for .safetensors checkpoints.
//
// The file is mapped once; the JSON header is parsed into a table of (name, dtype, shape, byte
// range); tensors are handed out as pointers into the mapping, so a loader can copy exactly the
// tensors (or the slices) one rank needs straight from the page cache to the device without ever
// holding the whole checkpoint in host memory, which matters for checkpoints sized for 180 GB
// GPUs. `rmlx_st_read` is a multi-threaded copy into a caller buffer (typically pinned memory).
//
// Native counterpart of the reference's safetensors loader
// (crates/rmlx-nn/src/safetensors_loader.rs:7-19,122-162: header parse, dtype table, MLX
// weight/scales/biases triplets are recognised one level up, in Python).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

struct Entry {
  std::string name, dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;
};

// Minimal JSON reader for the header: an object of objects whose values are strings, integers,
// arrays of integers, or (under "__metadata__") an object of strings.
class Json {
 public:
  Json(const char* p, size_t n) : p_(p), end_(p + n) {}
  bool fail = false;

  void ws() { while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_; }
  bool eat(char c) {
    ws();
    if (p_ < end_ && *p_ == c) { ++p_; return true; }
    return false;
  }
  bool peek(char c) { ws(); return p_ < end_ && *p_ == c; }
  std::string str() {
    std::string out;
    if (!eat('"')) { fail = true; return out; }
    while (p_ < end_ && *p_ != '"') {
      char c = *p_++;
      if (c == '\\' && p_ < end_) {
        char e = *p_++;
        switch (e) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {               // keep the escape as it is: tensor names are ASCII in practice
            out += "\\u";
            break;
          }
          default: out += e;        // \" \\ \/
        }
      } else {
        out += c;
      }
    }
    if (p_ >= end_) { fail = true; return out; }
    ++p_;
    return out;
  }
  int64_t integer() {
    ws();
    bool neg = false;
    if (p_ < end_ && *p_ == '-') { neg = true; ++p_; }
    if (p_ >= end_ || *p_ < '0' || *p_ > '9') { fail = true; return 0; }
    int64_t v = 0;
    while (p_ < end_ && *p_ >= '0' && *p_ <= '9') v = v * 10 + (*p_++ - '0');
    return neg ? -v : v;
  }
  // Skips any value (used for "__metadata__").
  void skip() {
    ws();
    if (p_ >= end_) { fail = true; return; }
    if (*p_ == '"') { str(); return; }
    if (*p_ == '{' || *p_ == '[') {
      const char open = *p_, close = open == '{' ? '}' : ']';
      ++p_;
      if (eat(close)) return;
      do {
        if (open == '{') { str(); if (!eat(':')) { fail = true; return; } }
        skip();
        if (fail) return;
      } while (eat(','));
      if (!eat(close)) fail = true;
      return;
    }
    while (p_ < end_ && *p_ != ',' && *p_ != '}' && *p_ != ']') ++p_;   // number / literal
  }

 private:
  const char* p_;
  const char* end_;
};

struct StFile {
  int fd = -1;
  char* map = nullptr;
  size_t size = 0, data_start = 0;
  std::vector<Entry> entries;
  std::unordered_map<std::string, int> index;
  ~StFile() {
    if (map) munmap(map, size);
    if (fd >= 0) close(fd);
  }
};

void set_err(char* err, int cap, const std::string& msg) {
  if (err && cap > 0) snprintf(err, static_cast<size_t>(cap), "%s", msg.c_str());
}

bool parse_header(StFile* f, const char* hdr, size_t n, std::string* why) {
  Json j(hdr, n);
  if (!j.eat('{')) { *why = "header is not a JSON object"; return false; }
  if (j.eat('}')) return true;
  do {
    std::string name = j.str();
    if (j.fail || !j.eat(':')) { *why = "bad key in header"; return false; }
    if (name == "__metadata__") {
      j.skip();
      if (j.fail) { *why = "bad __metadata__"; return false; }
      continue;
    }
    Entry e;
    e.name = name;
    if (!j.eat('{')) { *why = "tensor entry is not an object: " + name; return false; }
    do {
      std::string key = j.str();
      if (j.fail || !j.eat(':')) { *why = "bad field in " + name; return false; }
      if (key == "dtype") {
        e.dtype = j.str();
      } else if (key == "shape" || key == "data_offsets") {
        std::vector<int64_t> v;
        if (!j.eat('[')) { *why = "expected an array in " + name; return false; }
        if (!j.peek(']')) {
          do { v.push_back(j.integer()); } while (j.eat(','));
        }
        if (!j.eat(']')) { *why = "unterminated array in " + name; return false; }
        if (key == "shape") {
          e.shape = v;
        } else {
          if (v.size() != 2 || v[0] < 0 || v[1] < v[0]) { *why = "bad data_offsets in " + name; return false; }
          e.begin = static_cast<uint64_t>(v[0]);
          e.end = static_cast<uint64_t>(v[1]);
        }
      } else {
        j.skip();
      }
      if (j.fail) { *why = "malformed entry " + name; return false; }
    } while (j.eat(','));
    if (!j.eat('}')) { *why = "unterminated entry " + name; return false; }
    if (f->data_start + e.end > f->size) { *why = "tensor " + name + " runs past the end of the file"; return false; }
    f->index[e.name] = static_cast<int>(f->entries.size());
    f->entries.push_back(std::move(e));
  } while (j.eat(','));
  if (!j.eat('}')) { *why = "unterminated header"; return false; }
  return true;
}

}  // namespace

#define ST(h) static_cast<StFile*>(h)

extern "C" {

// Maps the file and parses its header. On failure returns nullptr and writes the reason to err.
void* rmlx_st_open(const char* path, char* err, int err_cap) {
  StFile* f = new StFile();
  f->fd = open(path, O_RDONLY);
  if (f->fd < 0) { set_err(err, err_cap, std::string("cannot open ") + path); delete f; return nullptr; }
  struct stat st;
  if (fstat(f->fd, &st) != 0 || st.st_size < 8) {
    set_err(err, err_cap, "file too small for a safetensors header"); delete f; return nullptr;
  }
  f->size = static_cast<size_t>(st.st_size);
  // private, writable mapping: nothing writes to it, but consumers that wrap the memory in a
  // tensor expect a writable buffer
  void* m = mmap(nullptr, f->size, PROT_READ | PROT_WRITE, MAP_PRIVATE, f->fd, 0);
  if (m == MAP_FAILED) { set_err(err, err_cap, "mmap failed"); delete f; return nullptr; }
  f->map = static_cast<char*>(m);
  uint64_t hdr_len = 0;
  memcpy(&hdr_len, f->map, 8);                       // little-endian u64
  if (hdr_len > f->size - 8) { set_err(err, err_cap, "header length exceeds the file"); delete f; return nullptr; }
  f->data_start = 8 + static_cast<size_t>(hdr_len);
  std::string why;
  if (!parse_header(f, f->map + 8, static_cast<size_t>(hdr_len), &why)) {
    set_err(err, err_cap, why); delete f; return nullptr;
  }
  return f;
}
void rmlx_st_close(void* h) { delete ST(h); }
int rmlx_st_count(void* h) { return static_cast<int>(ST(h)->entries.size()); }
int rmlx_st_find(void* h, const char* name) {
  auto it = ST(h)->index.find(name);
  return it == ST(h)->index.end() ? -1 : it->second;
}
const char* rmlx_st_name(void* h, int i) { return ST(h)->entries[i].name.c_str(); }
const char* rmlx_st_dtype(void* h, int i) { return ST(h)->entries[i].dtype.c_str(); }
int rmlx_st_ndim(void* h, int i) { return static_cast<int>(ST(h)->entries[i].shape.size()); }
void rmlx_st_shape(void* h, int i, int64_t* out) {
  const auto& s = ST(h)->entries[i].shape;
  for (size_t d = 0; d < s.size(); ++d) out[d] = s[d];
}
uint64_t rmlx_st_nbytes(void* h, int i) { return ST(h)->entries[i].end - ST(h)->entries[i].begin; }
void* rmlx_st_data(void* h, int i) { return ST(h)->map + ST(h)->data_start + ST(h)->entries[i].begin; }

// Copies nbytes of tensor i starting at byte `offset` into dst with up to `threads` threads
// (0 = choose). Returns 0, or -2 when the range is outside the tensor.
int rmlx_st_read(void* h, int i, void* dst, uint64_t offset, uint64_t nbytes, int threads) {
  const Entry& e = ST(h)->entries[i];
  if (offset > e.end - e.begin || nbytes > e.end - e.begin - offset) return -2;
  const char* src = ST(h)->map + ST(h)->data_start + e.begin + offset;
  constexpr uint64_t kChunk = 8ull << 20;            // below this one thread is as fast
  if (threads <= 0) threads = static_cast<int>(std::min<uint64_t>(8, std::max<unsigned>(1, std::thread::hardware_concurrency())));
  const uint64_t want = (nbytes + kChunk - 1) / kChunk;
  const int n = static_cast<int>(std::max<uint64_t>(1, std::min<uint64_t>(static_cast<uint64_t>(threads), want)));
  if (n == 1) {
    memcpy(dst, src, nbytes);
    return 0;
  }
  std::vector<std::thread> pool;
  const uint64_t per = (nbytes + n - 1) / n;
  for (int t = 0; t < n; ++t) {
    const uint64_t lo = per * t, hi = std::min(nbytes, lo + per);
    if (lo >= hi) break;
    pool.emplace_back([=] { memcpy(static_cast<char*>(dst) + lo, src + lo, hi - lo); });
  }
  for (auto& th : pool) th.join();
  return 0;
}

}  // extern "C"
