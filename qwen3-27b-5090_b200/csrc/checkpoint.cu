// Loader side of the path: NVFP4 projections read from a safetensors checkpoint straight into the buffers the GEMM
// kernels consume - codes [out][in / 2] (gate and up interleaved in blocks of 64 rows where asked), block scales
// swizzled into 512-byte atoms on the device, and the two tensor scales as floats.
//
// Two on-disk namings are understood, as by the reference's loader (engine/src/weights.cc:125-141, weights.h:71-75):
//   modelopt            <p>.weight        U8 [out][in/2]   <p>.weight_scale F8_E4M3 [out][in/16]
//                       <p>.weight_scale_2 F32 scalar       <p>.input_scale  F32 scalar
//   compressed-tensors  <p>.weight_packed U8 [out][in/2]   <p>.weight_scale F8_E4M3 [out][in/16]
//                       <p>.weight_global_scale = 1 / weight_scale_2    <p>.input_global_scale = 1 / input_scale
// A checkpoint is one .safetensors file or a directory of them (every shard's own header says what it holds).
//
// The upload: the file is read with pread into two pinned staging buffers in turn (the next piece is read while the
// previous one is copied), each piece goes to the device with one strided copy - for gate | up the stride skips the
// other half's blocks, which is the whole interleave (the reference's copy_glu, engine/src/weights.cc:218-234) - and
// the row-major scales land in a caller-provided device scratch from which q27b_swizzle_sf writes the atoms.
// Load-time code: it synchronises the stream, allocates its pinned staging once per checkpoint handle, and is not
// meant for a step.
#include <dirent.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/q27b200/capi.h"
#include "common.cuh"

namespace q27b {
namespace {

struct TensorEntry {
  std::string dtype;
  std::vector<int64_t> shape;
  int fd = -1;
  int64_t offset = 0, nbytes = 0;  // absolute offset in its file
};

// The few JSON forms a safetensors header uses: an object of objects with strings, integer arrays and (in
// "__metadata__") string values. A cursor over the text; every step checks bounds and reports by returning false.
struct HeaderScanner {
  const char* p;
  const char* end;
  void skip() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++;
  }
  bool eat(char c) {
    skip();
    if (p < end && *p == c) return p++, true;
    return false;
  }
  bool peek(char c) {
    skip();
    return p < end && *p == c;
  }
  bool string(std::string& out) {
    if (!eat('"')) return false;
    out.clear();
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (++p >= end) return false;
        switch (*p) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'u':  // (tensor names are ASCII in practice: keep the escape as it is written)
            out += "\\u";
            break;
          default: out += *p;
        }
        p++;
      } else {
        out += *p++;
      }
    }
    return p < end && *p++ == '"';
  }
  bool integer(int64_t& v) {
    skip();
    if (p >= end || *p < '0' || *p > '9') return false;
    v = 0;
    while (p < end && *p >= '0' && *p <= '9') {
      if (v > (INT64_MAX - 9) / 10) return false;
      v = v * 10 + (*p++ - '0');
    }
    return true;
  }
  bool int_array(std::vector<int64_t>& out) {
    if (!eat('[')) return false;
    out.clear();
    if (eat(']')) return true;
    do {
      int64_t v;
      if (!integer(v)) return false;
      out.push_back(v);
    } while (eat(','));
    return eat(']');
  }
  // any value, skipped (used for "__metadata__" and unknown keys)
  bool skip_value(int depth = 0) {
    skip();
    if (p >= end || depth > 16) return false;
    std::string s;
    if (*p == '"') return string(s);
    if (*p == '{' || *p == '[') {
      const char close = *p == '{' ? '}' : ']';
      const bool object = *p == '{';
      p++;
      if (eat(close)) return true;
      do {
        if (object && !(string(s) && eat(':'))) return false;
        if (!skip_value(depth + 1)) return false;
      } while (eat(','));
      return eat(close);
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']') p++;  // number, true, false, null
    return true;
  }
};

int64_t dtype_bytes(const std::string& d) {
  if (d == "U8" || d == "I8" || d == "F8_E4M3" || d == "F8_E5M2" || d == "BOOL") return 1;
  if (d == "BF16" || d == "F16" || d == "I16" || d == "U16") return 2;
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "F64" || d == "I64" || d == "U64") return 8;
  return 0;
}

bool read_fully(int fd, void* dst, int64_t len, int64_t off) {
  char* p = static_cast<char*>(dst);
  while (len > 0) {
    const ssize_t n = ::pread(fd, p, size_t(len), off);
    if (n <= 0) return false;
    p += n, off += n, len -= n;
  }
  return true;
}

constexpr size_t kStageBytes = size_t(32) << 20;

}  // namespace
}  // namespace q27b

struct q27b_ckpt {
  std::vector<int> fds;
  std::map<std::string, q27b::TensorEntry> tensors;
  // two pinned staging buffers with the event that says the copy out of each has completed (made on first upload)
  void* stage[2] = {nullptr, nullptr};
  cudaEvent_t drained[2] = {nullptr, nullptr};
  bool busy[2] = {false, false};
  int next = 0;
};

namespace q27b {
namespace {

int add_file(q27b_ckpt& c, const std::string& path) {
  const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
  Q27B_REQUIRE(fd >= 0, "ckpt_open: cannot open %s", path.c_str());
  c.fds.push_back(fd);
  struct stat st = {};
  Q27B_REQUIRE(::fstat(fd, &st) == 0 && st.st_size >= 8, "ckpt_open: %s is not a safetensors file", path.c_str());
  uint64_t hlen = 0;
  Q27B_REQUIRE(read_fully(fd, &hlen, 8, 0) && hlen >= 2 && hlen <= (uint64_t(100) << 20) && int64_t(8 + hlen) <= st.st_size,
               "ckpt_open: %s: bad header length", path.c_str());
  std::string text(size_t(hlen), '\0');
  Q27B_REQUIRE(read_fully(fd, &text[0], int64_t(hlen), 8), "ckpt_open: %s: short read of the header", path.c_str());
  const int64_t data0 = 8 + int64_t(hlen), data_bytes = st.st_size - data0;
  HeaderScanner s{text.data(), text.data() + text.size()};
  Q27B_REQUIRE(s.eat('{'), "ckpt_open: %s: header is not a JSON object", path.c_str());
  if (s.eat('}')) return 0;
  do {
    std::string name, key;
    Q27B_REQUIRE(s.string(name) && s.eat(':'), "ckpt_open: %s: malformed header", path.c_str());
    if (name == "__metadata__") {
      Q27B_REQUIRE(s.skip_value(), "ckpt_open: %s: malformed __metadata__", path.c_str());
      continue;
    }
    TensorEntry t;
    t.fd = fd;
    std::vector<int64_t> offs;
    Q27B_REQUIRE(s.eat('{'), "ckpt_open: %s: entry %s is not an object", path.c_str(), name.c_str());
    if (!s.peek('}')) {
      do {
        Q27B_REQUIRE(s.string(key) && s.eat(':'), "ckpt_open: %s: malformed entry %s", path.c_str(), name.c_str());
        bool ok = key == "dtype" ? s.string(t.dtype) : key == "shape" ? s.int_array(t.shape) : key == "data_offsets" ? s.int_array(offs) : s.skip_value();
        Q27B_REQUIRE(ok, "ckpt_open: %s: malformed %s of %s", path.c_str(), key.c_str(), name.c_str());
      } while (s.eat(','));
    }
    Q27B_REQUIRE(s.eat('}'), "ckpt_open: %s: malformed entry %s", path.c_str(), name.c_str());
    Q27B_REQUIRE(offs.size() == 2 && offs[0] <= offs[1] && offs[1] <= data_bytes, "ckpt_open: %s: %s lies outside the file", path.c_str(),
                 name.c_str());
    t.offset = data0 + offs[0], t.nbytes = offs[1] - offs[0];
    int64_t numel = 1;
    for (int64_t d : t.shape) {
      Q27B_REQUIRE(d >= 0 && (d == 0 || numel <= INT64_MAX / d), "ckpt_open: %s: bad shape of %s", path.c_str(), name.c_str());
      numel *= d;
    }
    const int64_t eb = dtype_bytes(t.dtype);
    Q27B_REQUIRE(eb == 0 || numel * eb == t.nbytes, "ckpt_open: %s: %s: %lld bytes for its shape and dtype %s", path.c_str(), name.c_str(),
                 (long long)t.nbytes, t.dtype.c_str());
    Q27B_REQUIRE(c.tensors.emplace(name, t).second, "ckpt_open: tensor %s appears twice", name.c_str());
  } while (s.eat(','));
  Q27B_REQUIRE(s.eat('}'), "ckpt_open: %s: malformed header (no closing brace)", path.c_str());
  return 0;
}

const TensorEntry* find(const q27b_ckpt* c, const std::string& name) {
  auto it = c->tensors.find(name);
  return it == c->tensors.end() ? nullptr : &it->second;
}

int read_scalar_f32(const q27b_ckpt* c, const std::string& name, bool inverse, float* out) {
  const TensorEntry* t = find(c, name);
  Q27B_REQUIRE(t, "ckpt: %s is missing", name.c_str());
  Q27B_REQUIRE(t->dtype == "F32" && t->nbytes == 4, "ckpt: %s: expected one F32 value", name.c_str());
  float v = 0.f;
  Q27B_REQUIRE(read_fully(t->fd, &v, 4, t->offset), "ckpt: %s: read failed", name.c_str());
  Q27B_REQUIRE(!inverse || v != 0.f, "ckpt: %s: a reciprocal scale of 0", name.c_str());
  *out = inverse ? 1.f / v : v;
  return 0;
}

// A staging buffer whose previous copy has drained.
int take_stage(q27b_ckpt* c, int* which) {
  if (!c->stage[0])
    for (int i = 0; i < 2; i++) {
      Q27B_CUDA(cudaMallocHost(&c->stage[i], kStageBytes));
      Q27B_CUDA(cudaEventCreateWithFlags(&c->drained[i], cudaEventDisableTiming));
    }
  const int i = c->next;
  c->next ^= 1;
  if (c->busy[i]) Q27B_CUDA(cudaEventSynchronize(c->drained[i]));
  c->busy[i] = false;
  *which = i;
  return 0;
}

// Rows [0, rows) of `row_bytes` each, from the file to dst. glu_half < 0: as they are; 0 / 1: block b of 64 rows goes
// to block 2 b + glu_half of the matrix that starts at dst.
int upload_rows(q27b_ckpt* c, const TensorEntry& t, int64_t rows, int64_t row_bytes, int glu_half, uint8_t* dst, cudaStream_t s) {
  const int64_t block_rows = glu_half >= 0 ? 64 : 1;
  int64_t step = int64_t(kStageBytes) / (row_bytes * block_rows) * block_rows;  // rows per piece: whole blocks
  Q27B_REQUIRE(step > 0, "ckpt: rows of %lld bytes do not fit the staging buffer", (long long)row_bytes);
  for (int64_t r0 = 0; r0 < rows; r0 += step) {
    const int64_t n = std::min(step, rows - r0);
    int b = 0;
    if (int rc = take_stage(c, &b)) return rc;
    Q27B_REQUIRE(read_fully(t.fd, c->stage[b], n * row_bytes, t.offset + r0 * row_bytes), "ckpt: read failed at row %lld", (long long)r0);
    if (glu_half < 0) {
      Q27B_CUDA(cudaMemcpyAsync(dst + r0 * row_bytes, c->stage[b], size_t(n * row_bytes), cudaMemcpyHostToDevice, s));
    } else if (int rc = q27b_copy_glu(dst, size_t(r0 * row_bytes), c->stage[b], size_t(n * row_bytes), size_t(64 * row_bytes), glu_half, s)) {
      return rc;
    }
    Q27B_CUDA(cudaEventRecord(c->drained[b], s));
    c->busy[b] = true;
  }
  return 0;
}

}  // namespace
}  // namespace q27b

using namespace q27b;

extern "C" {

int q27b_copy_glu(void* dst, size_t off, const void* host_src, size_t len, size_t block, int half, void* stream) {
  Q27B_REQUIRE(dst && host_src && block > 0 && (half == 0 || half == 1), "copy_glu: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* d = static_cast<char*>(dst);
  const char* src = static_cast<const char*>(host_src);
  auto place = [&](size_t o) { return d + (2 * (o / block) + size_t(half)) * block + o % block; };
  const size_t end = off + len;
  if (off % block && off < end) {  // the rest of a block that an earlier piece began
    const size_t n = std::min(end, (off / block + 1) * block) - off;
    Q27B_CUDA(cudaMemcpyAsync(place(off), src, n, cudaMemcpyHostToDevice, s));
    src += n, off += n;
  }
  if (const size_t whole = (end - off) / block) {  // whole blocks: one strided copy onto every other block
    Q27B_CUDA(cudaMemcpy2DAsync(place(off), 2 * block, src, block, block, whole, cudaMemcpyHostToDevice, s));
    src += whole * block, off += whole * block;
  }
  if (off < end) Q27B_CUDA(cudaMemcpyAsync(place(off), src, end - off, cudaMemcpyHostToDevice, s));
  return 0;
}

int q27b_ckpt_open(const char* path, q27b_ckpt** out) {
  Q27B_REQUIRE(path && out, "ckpt_open: null argument");
  *out = nullptr;
  q27b_ckpt* c = new q27b_ckpt();
  struct stat st = {};
  int rc = 0;
  if (::stat(path, &st) != 0) {
    rc = fail("ckpt_open: %s does not exist", path);
  } else if (S_ISDIR(st.st_mode)) {
    std::vector<std::string> files;
    if (DIR* d = ::opendir(path)) {
      while (dirent* e = ::readdir(d)) {
        const std::string n = e->d_name;
        if (n.size() > 12 && n.compare(n.size() - 12, 12, ".safetensors") == 0) files.push_back(std::string(path) + "/" + n);
      }
      ::closedir(d);
    }
    std::sort(files.begin(), files.end());
    if (files.empty()) rc = fail("ckpt_open: no .safetensors file in %s", path);
    for (size_t i = 0; rc == 0 && i < files.size(); i++) rc = add_file(*c, files[i]);
  } else {
    rc = add_file(*c, path);
  }
  if (rc) {
    q27b_ckpt_close(c);
    return rc;
  }
  *out = c;
  return 0;
}

void q27b_ckpt_close(q27b_ckpt* c) {
  if (!c) return;
  for (int fd : c->fds) ::close(fd);
  for (int i = 0; i < 2; i++) {
    if (c->drained[i]) {
      if (c->busy[i]) cudaEventSynchronize(c->drained[i]);
      cudaEventDestroy(c->drained[i]);
    }
    if (c->stage[i]) cudaFreeHost(c->stage[i]);
  }
  delete c;
}

int q27b_ckpt_count(const q27b_ckpt* c) { return c ? int(c->tensors.size()) : 0; }

int q27b_ckpt_tensor(const q27b_ckpt* c, const char* name, char* dtype, int dtype_cap, int64_t* shape, int shape_cap, int* ndim,
                     int64_t* nbytes) {
  Q27B_REQUIRE(c && name, "ckpt_tensor: null argument");
  const TensorEntry* t = find(c, name);
  if (!t) return 1;  // not in the checkpoint (not an error: the two namings are told apart this way)
  if (dtype && dtype_cap > 0) snprintf(dtype, size_t(dtype_cap), "%s", t->dtype.c_str());
  if (ndim) *ndim = int(t->shape.size());
  for (int i = 0; shape && i < shape_cap && i < int(t->shape.size()); i++) shape[i] = t->shape[i];
  if (nbytes) *nbytes = t->nbytes;
  return 0;
}

int q27b_ckpt_read(const q27b_ckpt* c, const char* name, int64_t begin, int64_t len, void* host_dst) {
  Q27B_REQUIRE(c && name && host_dst, "ckpt_read: null argument");
  const TensorEntry* t = find(c, name);
  Q27B_REQUIRE(t, "ckpt_read: %s is missing", name);
  Q27B_REQUIRE(begin >= 0 && len >= 0 && begin + len <= t->nbytes, "ckpt_read: %s: bytes [%lld, %lld) of %lld", name, (long long)begin,
               (long long)(begin + len), (long long)t->nbytes);
  Q27B_REQUIRE(read_fully(t->fd, host_dst, len, t->offset + begin), "ckpt_read: %s: read failed", name);
  return 0;
}

int q27b_ckpt_fp4_layer(const q27b_ckpt* c, const char* prefix, q27b_fp4_layer* info) {
  Q27B_REQUIRE(c && prefix && info, "ckpt_fp4_layer: null argument");
  const std::string p = prefix;
  const bool ct = find(c, p + ".weight_packed") != nullptr;
  const std::string wn = p + (ct ? ".weight_packed" : ".weight");
  const TensorEntry* w = find(c, wn);
  Q27B_REQUIRE(w, "ckpt_fp4_layer: %s has neither .weight nor .weight_packed", prefix);
  Q27B_REQUIRE(w->dtype == "U8" && w->shape.size() == 2 && w->shape[0] > 0 && w->shape[0] <= INT32_MAX && w->shape[1] > 0 &&
                   w->shape[1] <= INT32_MAX / 2,
               "ckpt_fp4_layer: %s: expected an NVFP4 matrix (U8 [out][in / 2])", wn.c_str());
  const int64_t out = w->shape[0], in = w->shape[1] * 2;
  Q27B_REQUIRE(in % 16 == 0, "ckpt_fp4_layer: %s: in = %lld is not a multiple of 16", prefix, (long long)in);
  const TensorEntry* sf = find(c, p + ".weight_scale");
  Q27B_REQUIRE(sf, "ckpt_fp4_layer: %s.weight_scale is missing", prefix);
  Q27B_REQUIRE(sf->dtype == "F8_E4M3" && sf->shape.size() == 2 && sf->shape[0] == out && sf->shape[1] == in / 16,
               "ckpt_fp4_layer: %s.weight_scale: expected F8_E4M3 [%lld][%lld]", prefix, (long long)out, (long long)(in / 16));
  info->out = int(out), info->in = int(in), info->compressed_tensors = ct ? 1 : 0;
  if (int rc = read_scalar_f32(c, p + (ct ? ".weight_global_scale" : ".weight_scale_2"), ct, &info->w_scale2)) return rc;
  return read_scalar_f32(c, p + (ct ? ".input_global_scale" : ".input_scale"), ct, &info->in_scale);
}

int q27b_ckpt_load_fp4(q27b_ckpt* c, const char* prefix, int glu_half, uint8_t* w, uint8_t* sf, void* scratch, size_t scratch_bytes,
                       void* stream) {
  Q27B_REQUIRE(c && prefix && w && sf && scratch, "ckpt_load_fp4: null argument");
  Q27B_REQUIRE(glu_half >= -1 && glu_half <= 1, "ckpt_load_fp4: glu_half is -1, 0 or 1");
  q27b_fp4_layer li = {};
  if (int rc = q27b_ckpt_fp4_layer(c, prefix, &li)) return rc;
  Q27B_REQUIRE(glu_half < 0 || li.out % 64 == 0, "ckpt_load_fp4: %s: gate | up interleave needs out %% 64 == 0 (out = %d)", prefix, li.out);
  const int kblocks = li.in / 16;
  Q27B_REQUIRE(scratch_bytes >= size_t(li.out) * size_t(kblocks), "ckpt_load_fp4: %s: scratch of %zu bytes, %zu needed", prefix, scratch_bytes,
               size_t(li.out) * size_t(kblocks));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const std::string p = prefix;
  const TensorEntry* wt = find(c, p + (li.compressed_tensors ? ".weight_packed" : ".weight"));
  const TensorEntry* st = find(c, p + ".weight_scale");
  if (int rc = upload_rows(c, *wt, li.out, li.in / 2, glu_half, w, s)) return rc;
  if (int rc = upload_rows(c, *st, li.out, kblocks, -1, static_cast<uint8_t*>(scratch), s)) return rc;
  if (int rc = q27b_swizzle_sf(static_cast<const uint8_t*>(scratch), li.out, kblocks, sf, glu_half, s)) return rc;
  Q27B_CUDA(cudaStreamSynchronize(s));  // the scratch and the staging buffers are the caller's again
  c->busy[0] = c->busy[1] = false;
  return 0;
}

}  // extern "C"
