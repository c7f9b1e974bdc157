// GGUF file reader and tensor upload (C ABI: the bpq4k_gguf_* entry points of include/bpq4k.h).
//
// Stands in for the reference's GGUFFile::open and metadata accessors
// (runtime/gguf_loader.cpp:14-182, runtime/gguf_loader.h:46-91) and for the K-quant part of its
// weight loading (pack + uploadKQWeight, runtime/model_runner.cpp:958-963, 1054-1061): the on-disk
// block format is the device format, so a Q4_K / Q5_K tensor goes from the file to HBM through a
// pinned double buffer without touching its bytes; Q6_K blocks are re-spaced on the device (to whole
// words per row as pack_q6k does, or to the padded 224-byte layout of the streaming kernel).
//
// Unlike the reference's reader every length read from the file is checked against the file size,
// so a truncated or corrupt file yields an error instead of a huge allocation.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <initializer_list>
#include <new>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../../include/bpq4k.h"
#include "kernels.h"

namespace {

enum MetaType : uint32_t {
    kU8 = 0, kI8 = 1, kU16 = 2, kI16 = 3, kU32 = 4, kI32 = 5, kF32 = 6, kBool = 7,
    kString = 8, kArray = 9, kU64 = 10, kI64 = 11, kF64 = 12,
};

struct MetaValue {
    uint32_t type = kString;        // scalar type, or kArray
    uint32_t elem_type = 0;         // arrays
    uint64_t u = 0;                 // unsigned / bool scalars
    int64_t i = 0;                  // signed scalars
    double f = 0.0;                 // float scalars
    std::string s;                  // string scalar
    std::vector<std::string> strs;  // string array
    std::vector<int64_t> ints;      // integer / bool arrays
    std::vector<double> floats;     // float arrays
    uint64_t count = 0;             // array length (also for arrays whose elements were skipped)
};

struct TensorInfo {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t shape[4] = {1, 1, 1, 1};
    uint32_t type = 0;
    uint64_t offset = 0;  // relative to data_offset
};

}  // namespace

struct bpq4k_gguf {
    std::string path;
    int fd = -1;
    uint64_t file_size = 0;
    uint32_t version = 0;
    uint64_t data_offset = 0;
    uint32_t alignment = 32;
    std::unordered_map<std::string, MetaValue> meta;
    std::vector<TensorInfo> tensors;
    std::unordered_map<std::string, uint64_t> index;
    std::string err = "no error";
    // pinned staging buffers of the upload path (allocated by the first upload, kept until close)
    static constexpr int kLanes = 4;
    static constexpr uint64_t kChunk = 8ull << 20;
    int staging_dev = -1;
    uint8_t* pinned[kLanes] = {nullptr, nullptr, nullptr, nullptr};
    cudaStream_t lane_stream[kLanes] = {nullptr, nullptr, nullptr, nullptr};
};

namespace {

// Sequential reader over the file with bounds checks.
struct Cursor {
    int fd;
    uint64_t pos = 0, size = 0;
    bool ok = true;
    bool read(void* dst, uint64_t n) {
        if (!ok || n > size - pos) return ok = false;
        uint8_t* p = static_cast<uint8_t*>(dst);
        uint64_t done = 0;
        while (done < n) {
            const ssize_t r = pread(fd, p + done, n - done, (off_t)(pos + done));
            if (r <= 0) return ok = false;
            done += (uint64_t)r;
        }
        pos += n;
        return true;
    }
    template <typename T>
    T get() {
        T v{};
        read(&v, sizeof(T));
        return v;
    }
    std::string str() {
        const uint64_t len = get<uint64_t>();
        if (!ok || len > size - pos) {
            ok = false;
            return std::string();
        }
        std::string s((size_t)len, '\0');
        read(&s[0], len);
        return s;
    }
};

bool read_scalar(Cursor& c, uint32_t type, MetaValue& v) {
    v.type = type;
    switch (type) {
        case kU8: v.u = c.get<uint8_t>(); break;
        case kI8: v.i = c.get<int8_t>(); break;
        case kU16: v.u = c.get<uint16_t>(); break;
        case kI16: v.i = c.get<int16_t>(); break;
        case kU32: v.u = c.get<uint32_t>(); break;
        case kI32: v.i = c.get<int32_t>(); break;
        case kF32: v.f = c.get<float>(); break;
        case kBool: v.u = c.get<uint8_t>() != 0; break;
        case kString: v.s = c.str(); break;
        case kU64: v.u = c.get<uint64_t>(); break;
        case kI64: v.i = c.get<int64_t>(); break;
        case kF64: v.f = c.get<double>(); break;
        default: return false;
    }
    return c.ok;
}

bool read_value(Cursor& c, uint32_t type, MetaValue& v, int depth) {
    if (type != kArray) return read_scalar(c, type, v);
    v.type = kArray;
    v.elem_type = c.get<uint32_t>();
    v.count = c.get<uint64_t>();
    if (!c.ok || v.count > c.size) return c.ok = false;  // every element takes at least a byte
    for (uint64_t k = 0; k < v.count; k++) {
        MetaValue e;
        if (v.elem_type == kArray) {
            if (depth > 4 || !read_value(c, kArray, e, depth + 1)) return c.ok = false;  // nested arrays are skipped
            continue;
        }
        if (!read_scalar(c, v.elem_type, e)) return false;
        switch (v.elem_type) {
            case kString: v.strs.push_back(std::move(e.s)); break;
            case kF32: case kF64: v.floats.push_back(e.f); break;
            case kU8: case kU16: case kU32: case kU64: case kBool: v.ints.push_back((int64_t)e.u); break;
            default: v.ints.push_back(e.i); break;
        }
    }
    return true;
}

// Bytes of a tensor of `n` elements of a GGML type whose rows hold `ne0` elements; 0 for a type this
// reader cannot size.
uint64_t tensor_bytes(uint32_t type, uint64_t n, uint64_t ne0) {
    struct TS { uint32_t type, block, bytes; };
    static const TS table[] = {{0, 1, 4},   {1, 1, 2},    {2, 32, 18},   {3, 32, 20},   {6, 32, 22},  {7, 32, 24},
                               {8, 32, 34}, {9, 32, 36},  {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176},
                               {14, 256, 210}, {20, 32, 18}, {23, 256, 136}, {24, 1, 1}, {25, 1, 2}, {26, 1, 4}, {27, 1, 8},
                               {28, 1, 8}, {30, 1, 2}};
    for (const TS& t : table)
        if (t.type == type) return (ne0 % t.block) ? 0 : n / t.block * t.bytes;
    return 0;
}

int gfail(bpq4k_gguf* g, int status, const std::string& msg) {
    if (g) g->err = msg;
    return status;
}

// Q6_K: file-format blocks (210 bytes, rows contiguous) -> rows `out_row_bytes` apart with blocks
// `out_block_bytes` apart (210: pack_q6k's layout, 224: the padded layout); the gaps are zeroed.
__global__ void __launch_bounds__(256) q6k_respace_kernel(const uint8_t* __restrict__ raw, uint64_t n_blocks_total, uint32_t nb,
                                                          uint8_t* __restrict__ out, uint64_t out_row_bytes,
                                                          uint32_t out_block_bytes) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warps = (uint64_t)gridDim.x * (blockDim.x >> 5);
    for (uint64_t blk = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); blk < n_blocks_total; blk += warps) {
        const uint64_t row = blk / nb;
        const uint32_t b = (uint32_t)(blk - row * nb);
        const uint16_t* src = reinterpret_cast<const uint16_t*>(raw + blk * 210u);  // blocks are 2-byte aligned
        uint16_t* dst = reinterpret_cast<uint16_t*>(out + row * out_row_bytes + (uint64_t)b * out_block_bytes);
        for (uint32_t i = lane; i < out_block_bytes / 2u; i += 32u) dst[i] = i < 105u ? src[i] : (uint16_t)0;
        if (b == nb - 1u) {  // tail of the row (pack_q6k pads rows to a whole word)
            uint8_t* tail = out + row * out_row_bytes + (uint64_t)nb * out_block_bytes;
            for (uint64_t i = lane; i < out_row_bytes - (uint64_t)nb * out_block_bytes; i += 32u) tail[i] = 0;
        }
    }
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

int bpq4k_gguf_open(const char* path, bpq4k_gguf_t* out) {
    if (!path || !out) return BPQ4K_ERR_INVALID_ARG;
    *out = nullptr;
    bpq4k_gguf* g = new (std::nothrow) bpq4k_gguf();
    if (!g) return BPQ4K_ERR_ALLOC;
    g->path = path;
    g->fd = ::open(path, O_RDONLY);
    struct stat sb;
    if (g->fd < 0 || fstat(g->fd, &sb) != 0) {
        if (g->fd >= 0) ::close(g->fd);
        delete g;
        return BPQ4K_ERR_INVALID_ARG;
    }
    g->file_size = (uint64_t)sb.st_size;
    Cursor c{g->fd, 0, g->file_size};
    auto bad = [&](int status) {
        ::close(g->fd);
        delete g;
        return status;
    };
    if (c.get<uint32_t>() != 0x46554747u || !c.ok) return bad(BPQ4K_ERR_UNSUPPORTED);  // "GGUF"
    g->version = c.get<uint32_t>();
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (!c.ok || g->version < 2 || n_tensors > g->file_size || n_kv > g->file_size) return bad(BPQ4K_ERR_UNSUPPORTED);
    for (uint64_t k = 0; k < n_kv; k++) {
        std::string key = c.str();
        const uint32_t vtype = c.get<uint32_t>();
        MetaValue v;
        if (!c.ok || !read_value(c, vtype, v, 0)) return bad(BPQ4K_ERR_UNSUPPORTED);
        g->meta[key] = std::move(v);
    }
    g->tensors.resize((size_t)n_tensors);
    for (uint64_t t = 0; t < n_tensors; t++) {
        TensorInfo& ti = g->tensors[(size_t)t];
        ti.name = c.str();
        ti.n_dims = c.get<uint32_t>();
        if (!c.ok || ti.n_dims > 4) return bad(BPQ4K_ERR_UNSUPPORTED);
        for (uint32_t d = 0; d < ti.n_dims; d++) ti.shape[d] = c.get<uint64_t>();
        ti.type = c.get<uint32_t>();
        ti.offset = c.get<uint64_t>();
        if (!c.ok) return bad(BPQ4K_ERR_UNSUPPORTED);
        g->index[ti.name] = t;
    }
    // The tensor data starts at the next multiple of the alignment (general.alignment, 32 when absent;
    // the reference always uses 32, runtime/gguf_loader.cpp:131-132).
    auto it = g->meta.find("general.alignment");
    if (it != g->meta.end() && it->second.type == kU32 && it->second.u >= 1 && it->second.u <= (1u << 20)) g->alignment = (uint32_t)it->second.u;
    g->data_offset = (c.pos + g->alignment - 1) / g->alignment * g->alignment;
    *out = g;
    return BPQ4K_OK;
}

int bpq4k_gguf_close(bpq4k_gguf_t g) {
    if (!g) return BPQ4K_ERR_INVALID_ARG;
    if (g->fd >= 0) ::close(g->fd);
    if (g->staging_dev >= 0) {
        int prev = -1;
        cudaGetDevice(&prev);
        if (prev != g->staging_dev) cudaSetDevice(g->staging_dev);
        for (int i = 0; i < bpq4k_gguf::kLanes; i++) {
            if (g->lane_stream[i]) cudaStreamDestroy(g->lane_stream[i]);
            if (g->pinned[i]) cudaFreeHost(g->pinned[i]);
        }
        if (prev >= 0 && prev != g->staging_dev) cudaSetDevice(prev);
    }
    delete g;
    return BPQ4K_OK;
}

const char* bpq4k_gguf_last_error(bpq4k_gguf_t g) { return g ? g->err.c_str() : "null file"; }
uint32_t bpq4k_gguf_version(bpq4k_gguf_t g) { return g ? g->version : 0; }
uint64_t bpq4k_gguf_n_tensors(bpq4k_gguf_t g) { return g ? g->tensors.size() : 0; }
uint64_t bpq4k_gguf_data_offset(bpq4k_gguf_t g) { return g ? g->data_offset : 0; }

int bpq4k_gguf_has_key(bpq4k_gguf_t g, const char* key) { return g && key && g->meta.count(key) ? 1 : 0; }

// getU32 of the reference (runtime/gguf_loader.cpp:146-169): any integer scalar, or the maximum of an
// integer array; `def` otherwise.
uint32_t bpq4k_gguf_get_u32(bpq4k_gguf_t g, const char* key, uint32_t def) {
    if (!g || !key) return def;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return def;
    const MetaValue& v = it->second;
    switch (v.type) {
        case kU8: case kU16: case kU32: case kU64: return (uint32_t)v.u;
        case kI8: case kI16: case kI32: case kI64: return (uint32_t)v.i;
        case kArray:
            if ((v.elem_type == kI32 || v.elem_type == kU32) && !v.ints.empty()) {
                int32_t m = (int32_t)v.ints[0];
                for (int64_t x : v.ints)
                    if ((int32_t)x > m) m = (int32_t)x;
                return (uint32_t)m;
            }
            return def;
        default: return def;
    }
}

float bpq4k_gguf_get_f32(bpq4k_gguf_t g, const char* key, float def) {
    if (!g || !key) return def;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return def;
    return (it->second.type == kF32 || it->second.type == kF64) ? (float)it->second.f : def;
}

int bpq4k_gguf_get_bool(bpq4k_gguf_t g, const char* key, int def) {
    if (!g || !key) return def;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.type != kBool) return def;
    return it->second.u ? 1 : 0;
}

// String value (or element `index` of a string array when index >= 0) copied into buf; returns the
// string's length, or -1 when the key is absent or not a string.
int64_t bpq4k_gguf_get_string(bpq4k_gguf_t g, const char* key, int64_t index, char* buf, uint64_t cap) {
    if (!g || !key) return -1;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return -1;
    const MetaValue& v = it->second;
    const std::string* s = nullptr;
    if (index < 0 && v.type == kString) s = &v.s;
    if (index >= 0 && v.type == kArray && v.elem_type == kString && (uint64_t)index < v.strs.size()) s = &v.strs[(size_t)index];
    if (!s) return -1;
    if (buf && cap) {
        const uint64_t n = s->size() < cap - 1 ? s->size() : cap - 1;
        std::memcpy(buf, s->data(), n);
        buf[n] = '\0';
    }
    return (int64_t)s->size();
}

// Length of an array value (any element type); -1 when the key is absent or not an array.
int64_t bpq4k_gguf_array_length(bpq4k_gguf_t g, const char* key) {
    if (!g || !key) return -1;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.type != kArray) return -1;
    return (int64_t)it->second.count;
}

// Integer / bool array elements [first, first+n) as int32 (getI32Array / getBoolArray of the reference).
int bpq4k_gguf_get_i32_array(bpq4k_gguf_t g, const char* key, uint64_t first, uint64_t n, int32_t* out) {
    if (!g || !key || (!out && n)) return BPQ4K_ERR_INVALID_ARG;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.type != kArray || first + n > it->second.ints.size()) return BPQ4K_ERR_INVALID_ARG;
    for (uint64_t k = 0; k < n; k++) out[k] = (int32_t)it->second.ints[(size_t)(first + k)];
    return BPQ4K_OK;
}

int bpq4k_gguf_find_tensor(bpq4k_gguf_t g, const char* name, uint64_t* index) {
    if (!g || !name) return BPQ4K_ERR_INVALID_ARG;
    auto it = g->index.find(name);
    if (it == g->index.end()) return gfail(g, BPQ4K_ERR_INVALID_ARG, std::string("no tensor named ") + name);
    if (index) *index = it->second;
    return BPQ4K_OK;
}

int bpq4k_gguf_tensor_info(bpq4k_gguf_t g, uint64_t index, const char** name, uint32_t* n_dims, uint64_t shape[4],
                           uint32_t* type, uint64_t* offset, uint64_t* n_bytes) {
    if (!g || index >= g->tensors.size()) return BPQ4K_ERR_INVALID_ARG;
    const TensorInfo& t = g->tensors[(size_t)index];
    if (name) *name = t.name.c_str();
    if (n_dims) *n_dims = t.n_dims;
    if (shape)
        for (int d = 0; d < 4; d++) shape[d] = t.shape[d];
    if (type) *type = t.type;
    if (offset) *offset = t.offset;
    if (n_bytes) {
        uint64_t n = 1;
        for (uint32_t d = 0; d < t.n_dims; d++) n *= t.shape[d];
        *n_bytes = tensor_bytes(t.type, n, t.shape[0]);
    }
    return BPQ4K_OK;
}

// Raw bytes [first, first+n) of a tensor into host memory.
int bpq4k_gguf_read_tensor(bpq4k_gguf_t g, uint64_t index, uint64_t first, uint64_t n, void* dst_host) {
    if (!g || index >= g->tensors.size() || (!dst_host && n)) return BPQ4K_ERR_INVALID_ARG;
    const TensorInfo& t = g->tensors[(size_t)index];
    const uint64_t start = g->data_offset + t.offset + first;
    if (start > g->file_size || n > g->file_size - start) return gfail(g, BPQ4K_ERR_INVALID_ARG, "tensor data lies outside the file");
    Cursor c{g->fd, start, g->file_size};
    return c.read(dst_host, n) ? BPQ4K_OK : gfail(g, BPQ4K_ERR_INVALID_ARG, "short read");
}

// File-format Q6_K blocks already on the device (N rows of K/256 blocks of 210 bytes, no padding) ->
// the layout `layout_qtype` asks for (BPQ4K_TYPE_Q6_K: pack_q6k's word-padded rows; BPQ4K_TYPE_Q6_K_PADDED:
// 224-byte blocks).  `out_dev` holds N * bpq4k_kq_row_stride_words(layout_qtype, K) words.
int bpq4k_kq_respace_device(bpq4k_handle_t h, int layout_qtype, const void* raw_dev, uint32_t N, uint32_t K, void* out_dev,
                            void* stream) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (layout_qtype != BPQ4K_TYPE_Q6_K && layout_qtype != BPQ4K_TYPE_Q6_K_PADDED) return BPQ4K_ERR_UNSUPPORTED;
    if (K == 0 || K % 256 != 0) return BPQ4K_ERR_UNSUPPORTED;
    if (N == 0) return BPQ4K_OK;
    if (!raw_dev || !out_dev || (reinterpret_cast<uintptr_t>(raw_dev) & 1u) || (reinterpret_cast<uintptr_t>(out_dev) & 3u))
        return BPQ4K_ERR_INVALID_ARG;
    const uint32_t nb = K / 256;
    const uint64_t nblocks = (uint64_t)N * nb;
    uint64_t ctas = (nblocks + 7) / 8;
    if (ctas > 148ull * 32) ctas = 148ull * 32;
    int prev = -1;
    cudaGetDevice(&prev);
    const int dev = bpq4k_device_index(h);
    if (dev != prev) cudaSetDevice(dev);
    q6k_respace_kernel<<<(unsigned)ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(raw_dev), nblocks, nb, static_cast<uint8_t*>(out_dev),
        (uint64_t)bpq4k_kq_row_stride_words(layout_qtype, K) * 4u, bpq4k_kq_block_bytes(layout_qtype));
    const cudaError_t e = cudaGetLastError();
    if (dev != prev && prev >= 0) cudaSetDevice(prev);
    return e == cudaSuccess ? BPQ4K_OK : BPQ4K_ERR_CUDA;
}

// Load Q4_K / Q5_K / Q6_K tensors into device memory in the layout the matmul entry points take.
// layout_qtype: 0 = the reference's packed layout of the tensors' own type; BPQ4K_TYPE_Q6_K_PADDED for
// Q6_K tensors selects the padded layout.  Rows of a tensor = product of all dims but the first (expert
// stacks are row-stacked matrices).  Several tensors of one type and one K are concatenated by rows into
// ONE allocation -- the reference's fuseKQ (runtime/model_runner.cpp:1002-1012) done by where the bytes
// land instead of by a host-side copy.  The copy runs through four pinned 8 MB buffers, each filled by
// its own thread and sent on its own stream, so that file reads overlap each other and the transfers;
// the call returns when the tensors are resident.
int bpq4k_gguf_upload_fused(bpq4k_handle_t h, bpq4k_gguf_t g, const uint64_t* indices, uint32_t count, int layout_qtype,
                            void** w_dev, int* qtype_out, uint32_t* N_out, uint32_t* K_out, uint32_t* rowStrideWords_out) {
    if (!h || !g || !w_dev || !indices || count == 0) return BPQ4K_ERR_INVALID_ARG;
    *w_dev = nullptr;
    for (uint32_t i = 0; i < count; i++)
        if (indices[i] >= g->tensors.size()) return BPQ4K_ERR_INVALID_ARG;
    const TensorInfo& t0 = g->tensors[(size_t)indices[0]];
    if (t0.type != BPQ4K_TYPE_Q4_K && t0.type != BPQ4K_TYPE_Q5_K && t0.type != BPQ4K_TYPE_Q6_K)
        return gfail(g, BPQ4K_ERR_UNSUPPORTED, t0.name + ": not a Q4_K, Q5_K or Q6_K tensor");
    int layout = layout_qtype ? layout_qtype : (int)t0.type;
    if (layout != (int)t0.type && !(layout == BPQ4K_TYPE_Q6_K_PADDED && t0.type == BPQ4K_TYPE_Q6_K))
        return gfail(g, BPQ4K_ERR_INVALID_ARG, t0.name + ": the requested layout does not belong to the tensor's type");
    const uint64_t K = t0.shape[0];
    if (t0.n_dims < 1 || K == 0 || K % 256 != 0 || K > 0xFFFFFFFFull)
        return gfail(g, BPQ4K_ERR_UNSUPPORTED, t0.name + ": shape not supported (rows of a multiple of 256 weights)");
    const uint32_t nb = (uint32_t)(K / 256);
    const uint32_t file_bb = bpq4k_kq_block_bytes((int)t0.type);
    uint64_t N = 0;
    std::vector<uint64_t> rows(count);
    for (uint32_t i = 0; i < count; i++) {
        const TensorInfo& t = g->tensors[(size_t)indices[i]];
        if (t.type != t0.type || t.shape[0] != K)
            return gfail(g, BPQ4K_ERR_INVALID_ARG, t.name + ": tensors fused by rows need one type and one row length");
        uint64_t n = 1;
        for (uint32_t d = 1; d < t.n_dims; d++) n *= t.shape[d];
        const uint64_t bytes = n * nb * file_bb, start = g->data_offset + t.offset;
        if (n == 0 || start > g->file_size || bytes > g->file_size - start)
            return gfail(g, BPQ4K_ERR_INVALID_ARG, t.name + ": data lies outside the file");
        rows[i] = n;
        N += n;
    }
    if (N > 0xFFFFFFFFull) return gfail(g, BPQ4K_ERR_UNSUPPORTED, t0.name + ": more than 2^32 rows");
    const uint64_t raw_bytes = N * nb * file_bb;
    const uint32_t rs = bpq4k_kq_row_stride_words(layout, (uint32_t)K);
    const uint64_t out_bytes = N * (uint64_t)rs * 4u;
    const bool respace = t0.type == BPQ4K_TYPE_Q6_K;  // Q4_K / Q5_K: file bytes are the device bytes

    int dev_prev = -1;
    cudaGetDevice(&dev_prev);
    const int dev = bpq4k_device_index(h);
    void* out = nullptr;
    if (dev >= 0 && dev != dev_prev) cudaSetDevice(dev);
    auto restore = [&]() {
        if (dev >= 0 && dev != dev_prev && dev_prev >= 0) cudaSetDevice(dev_prev);
    };
    void* raw_dev = nullptr;
    int status = BPQ4K_OK;
    constexpr int kLanes = bpq4k_gguf::kLanes;
    constexpr uint64_t kChunk = bpq4k_gguf::kChunk;
    // staging: kLanes pinned buffers with a stream each, created once per file handle
    if (g->staging_dev != dev) {
        if (g->staging_dev >= 0) {
            restore();
            return gfail(g, BPQ4K_ERR_INVALID_ARG, "this file handle already uploads to another device");
        }
        bool ok = true;
        for (int i = 0; i < kLanes && ok; i++)
            ok = cudaHostAlloc((void**)&g->pinned[i], kChunk, cudaHostAllocDefault) == cudaSuccess &&
                 cudaStreamCreateWithFlags(&g->lane_stream[i], cudaStreamNonBlocking) == cudaSuccess;
        g->staging_dev = dev;  // close() releases whatever was created
        if (!ok) {
            cudaGetLastError();
            restore();
            return gfail(g, BPQ4K_ERR_ALLOC, t0.name + ": staging allocation failed");
        }
    }
    if (cudaMalloc(&out, out_bytes ? out_bytes : 16) != cudaSuccess) {
        cudaGetLastError();
        restore();
        return gfail(g, BPQ4K_ERR_ALLOC, t0.name + ": device allocation failed");
    }
    raw_dev = out;
    if (respace && cudaMalloc(&raw_dev, raw_bytes) != cudaSuccess) {
        cudaGetLastError();
        raw_dev = nullptr;
        status = gfail(g, BPQ4K_ERR_ALLOC, t0.name + ": device allocation failed");
    }
    auto cleanup = [&]() {
        if (raw_dev && raw_dev != out) cudaFree(raw_dev);
    };
    if (status == BPQ4K_OK) {
        // One list of (file position, device position, bytes) chunks over all tensors; lane i takes chunks
        // i, i+kLanes, ...: read into its pinned buffer, copy on its stream, wait, next chunk -- file reads of one
        // lane overlap the transfers of the others
        struct Piece { uint64_t file_pos, dev_off, n; };
        std::vector<Piece> pieces;
        uint64_t dev_off = 0;
        for (uint32_t i = 0; i < count; i++) {
            const TensorInfo& t = g->tensors[(size_t)indices[i]];
            const uint64_t bytes = rows[i] * nb * file_bb, start = g->data_offset + t.offset;
            for (uint64_t off = 0; off < bytes; off += kChunk)
                pieces.push_back({start + off, dev_off + off, bytes - off < kChunk ? bytes - off : kChunk});
            dev_off += bytes;
        }
        int lane_status[kLanes] = {0, 0, 0, 0};
        auto work = [&](int lane) {
            cudaSetDevice(dev);
            for (size_t ch = (size_t)lane; ch < pieces.size(); ch += kLanes) {
                const Piece& pc = pieces[ch];
                Cursor c{g->fd, pc.file_pos, g->file_size};
                if (!c.read(g->pinned[lane], pc.n)) {
                    lane_status[lane] = 1;
                    return;
                }
                if (cudaMemcpyAsync(static_cast<uint8_t*>(raw_dev) + pc.dev_off, g->pinned[lane], pc.n, cudaMemcpyHostToDevice,
                                    g->lane_stream[lane]) != cudaSuccess ||
                    cudaStreamSynchronize(g->lane_stream[lane]) != cudaSuccess) {
                    lane_status[lane] = 2;
                    return;
                }
            }
        };
        std::vector<std::thread> pool;
        const int used = pieces.size() < (size_t)kLanes ? (int)pieces.size() : kLanes;
        for (int i = 1; i < used; i++) pool.emplace_back(work, i);
        if (used > 0) work(0);
        for (auto& th : pool) th.join();
        for (int i = 0; i < kLanes; i++) {
            if (lane_status[i] == 1) status = gfail(g, BPQ4K_ERR_INVALID_ARG, t0.name + ": short read");
            if (lane_status[i] == 2) {
                cudaGetLastError();
                status = gfail(g, BPQ4K_ERR_CUDA, t0.name + ": copy to the device failed");
            }
        }
    }
    cudaStream_t st = g->lane_stream[0];
    if (status == BPQ4K_OK && respace) {
        const uint64_t nblocks = N * nb;
        uint64_t ctas = (nblocks + 7) / 8;
        if (ctas > 148ull * 32) ctas = 148ull * 32;
        q6k_respace_kernel<<<(unsigned)ctas, 256, 0, st>>>(static_cast<const uint8_t*>(raw_dev), nblocks, nb, static_cast<uint8_t*>(out),
                                                         (uint64_t)rs * 4u, bpq4k_kq_block_bytes(layout));
        if (cudaGetLastError() != cudaSuccess) status = gfail(g, BPQ4K_ERR_CUDA, t0.name + ": re-spacing kernel failed to launch");
    }
    if (cudaStreamSynchronize(st) != cudaSuccess && status == BPQ4K_OK) {
        cudaGetLastError();
        status = gfail(g, BPQ4K_ERR_CUDA, t0.name + ": upload failed");
    }
    cleanup();
    if (status != BPQ4K_OK) {
        cudaFree(out);
        restore();
        return status;
    }
    restore();
    *w_dev = out;
    if (qtype_out) *qtype_out = layout;
    if (N_out) *N_out = (uint32_t)N;
    if (K_out) *K_out = (uint32_t)K;
    if (rowStrideWords_out) *rowStrideWords_out = rs;
    return BPQ4K_OK;
}

int bpq4k_gguf_upload_tensor(bpq4k_handle_t h, bpq4k_gguf_t g, uint64_t index, int layout_qtype, void** w_dev,
                             int* qtype_out, uint32_t* N_out, uint32_t* K_out, uint32_t* rowStrideWords_out) {
    return bpq4k_gguf_upload_fused(h, g, &index, 1, layout_qtype, w_dev, qtype_out, N_out, K_out, rowStrideWords_out);
}

// ---- model configuration and the per-layer K-quant tensors ---------------------------------------

namespace {
bool has_tensor(bpq4k_gguf* g, const std::string& name) { return g->index.count(name) != 0; }
bool is_kquant(uint32_t type) { return type == BPQ4K_TYPE_Q4_K || type == BPQ4K_TYPE_Q5_K || type == BPQ4K_TYPE_Q6_K; }
}  // namespace

// extractModelConfig (runtime/gguf_loader.cpp:184-317), field for field.
int bpq4k_gguf_model_config(bpq4k_gguf_t g, bpq4k_model_config* c, uint8_t* layer_attn_types, uint32_t cap) {
    if (!g || !c) return BPQ4K_ERR_INVALID_ARG;
    std::memset(c, 0, sizeof(*c));
    auto str = [&](const std::string& key, const char* def) -> std::string {
        auto it = g->meta.find(key);
        return it != g->meta.end() && it->second.type == kString ? it->second.s : std::string(def);
    };
    auto u32 = [&](const std::string& key, uint32_t def = 0) { return bpq4k_gguf_get_u32(g, key.c_str(), def); };
    auto f32 = [&](const std::string& key, float def) { return bpq4k_gguf_get_f32(g, key.c_str(), def); };
    const std::string a = str("general.architecture", "llama");
    std::snprintf(c->arch, sizeof(c->arch), "%s", a.c_str());
    c->nLayer = u32(a + ".block_count");
    c->nEmbd = u32(a + ".embedding_length");
    c->intermediateSize = u32(a + ".feed_forward_length");
    c->nHead = u32(a + ".attention.head_count");
    c->nKvHeads = u32(a + ".attention.head_count_kv", c->nHead);
    c->rmsNormEps = f32(a + ".attention.layer_norm_rms_epsilon", 1e-6f);
    c->ropeTheta = f32(a + ".rope.freq_base", 1000000.0f);
    c->tieWordEmbeddings = g->meta.count("output.weight") ? 0 : 1;  // the reference asks the metadata, not the tensor list
    const uint32_t dense_head = c->nHead > 0 ? c->nEmbd / c->nHead : 0;
    c->kvHeadDim = u32(a + ".attention.key_length", dense_head);
    c->headDim = c->kvHeadDim > 0 ? c->kvHeadDim : dense_head;
    {
        auto it = g->index.find("token_embd.weight");
        if (it != g->index.end()) {
            const TensorInfo& t = g->tensors[(size_t)it->second];
            c->nVocab = (uint32_t)(t.n_dims >= 2 ? t.shape[1] : t.shape[0]);
        }
    }
    c->hasQkNorm = has_tensor(g, "blk.0.attn_q_norm.weight");
    for (uint32_t i = 1; !c->hasQkNorm && i < c->nLayer; i++)
        c->hasQkNorm = has_tensor(g, "blk." + std::to_string(i) + ".attn_q_norm.weight");
    const bool gemma = a == "gemma" || a == "gemma2" || a == "gemma3" || a == "gemma4";
    c->activation = gemma ? 1 : 0;
    c->embeddingScale = gemma ? sqrtf((float)c->nEmbd) : 0.0f;
    c->logitSoftcap = f32(a + ".final_logit_softcapping", 0.0f);
    c->slidingWindow = u32(a + ".attention.sliding_window", 0);
    c->nLayerAttnTypes = 0;
    if (c->slidingWindow > 0 && c->nLayer > 0) {
        c->nLayerAttnTypes = c->nLayer;
        const MetaValue* pattern = nullptr;
        if (a == "gemma4") {
            auto it = g->meta.find(a + ".attention.sliding_window_pattern");
            if (it != g->meta.end() && it->second.type == kArray && it->second.elem_type == kBool &&
                it->second.ints.size() == c->nLayer)
                pattern = &it->second;
        }
        for (uint32_t i = 0; i < c->nLayer && layer_attn_types && i < cap; i++) {
            uint8_t sliding = 0;  // Global unless the architecture says otherwise
            if (a == "gemma2") sliding = (i % 2 == 0);
            if (a == "gemma3") sliding = ((i + 1) % 6 != 0);
            if (a == "gemma4") sliding = pattern ? (pattern->ints[i] != 0) : ((i + 1) % 6 != 0);
            layer_attn_types[i] = sliding;
        }
    }
    c->sharedKvLayers = u32(a + ".attention.shared_kv_layers", 0);
    c->pleSize = u32(a + ".embedding_length_per_layer_input", 0);
    c->hasSandwichNorm = has_tensor(g, "blk.0.post_norm.weight") || has_tensor(g, "blk.0.attn_post_norm.weight") ||
                         has_tensor(g, "blk.0.post_attention_norm.weight");
    c->hasMtp = has_tensor(g, "mtp.0.blk.0.attn_q.weight") || has_tensor(g, "mtp.0.enorm.weight");
    if (!c->hasMtp) {
        const uint32_t nextn = u32(a + ".nextn_predict_layers", 0);
        if (nextn > 0) {
            c->hasMtp = 1;
            c->mtpNumLayers = nextn;
        }
    }
    c->numExperts = u32(a + ".expert_count", 0);
    c->numExpertsPerTok = u32(a + ".expert_used_count", 0);
    c->moeIntermediateSize = u32(a + ".expert_feed_forward_length", 0);
    c->moeSharedIntermediateSize = u32(a + ".expert_shared_feed_forward_length", c->moeIntermediateSize);
    c->ssmInnerSize = u32(a + ".ssm.inner_size", 0);
    c->ssmStateSize = u32(a + ".ssm.state_size", 0);
    c->ssmConvKernel = u32(a + ".ssm.conv_kernel", 0);
    c->ssmGroupCount = u32(a + ".ssm.group_count", 0);
    c->ssmTimeStepRank = u32(a + ".ssm.time_step_rank", 0);
    c->fullAttentionInterval = u32(a + ".full_attention_interval", 0);
    c->ropeSections[0] = 11, c->ropeSections[1] = 11, c->ropeSections[2] = 10, c->ropeSections[3] = 0;
    {
        auto it = g->meta.find(a + ".rope.dimension_sections");
        if (it != g->meta.end() && it->second.type == kArray && it->second.elem_type == kI32 && it->second.ints.size() >= 4)
            for (int i = 0; i < 4; i++) c->ropeSections[i] = (int32_t)it->second.ints[(size_t)i];
    }
    return BPQ4K_OK;
}

// The loader's quantisation probe (runtime/model_runner.cpp:1014-1049): the type of the first primary weight
// tensor found, and whether attn_q, ffn_gate and ffn_down of layer 0 all carry that one K-quant type.
int bpq4k_gguf_weight_format(bpq4k_gguf_t g, int* qtype, int* uniform_kquant) {
    if (!g || !qtype || !uniform_kquant) return BPQ4K_ERR_INVALID_ARG;
    *qtype = -1;
    for (const char* name : {"blk.0.attn_q.weight", "blk.0.attn_qkv.weight", "blk.0.ffn_gate.weight", "blk.0.ffn_down.weight"}) {
        auto it = g->index.find(name);
        if (it != g->index.end()) {
            *qtype = (int)g->tensors[(size_t)it->second].type;
            break;
        }
    }
    bool same = true;
    for (const char* name : {"blk.0.attn_q.weight", "blk.0.ffn_gate.weight", "blk.0.ffn_down.weight"}) {
        auto it = g->index.find(name);
        if (it == g->index.end()) continue;
        const uint32_t t = g->tensors[(size_t)it->second].type;
        if (!is_kquant(t) || (int)t != *qtype) same = false;
    }
    *uniform_kquant = same && *qtype >= 0 && is_kquant((uint32_t)*qtype) ? 1 : 0;
    return BPQ4K_OK;
}

// One transformer layer's projection weights onto the device with the loader's fusion rules
// (runtime/model_runner.cpp:1223-1370): Q+K+V concatenated by rows into one tensor (or a file's pre-fused
// attn_qkv taken as it is), attn_output, gate+up concatenated, ffn_down.  A group is fused when all its members
// are K-quant tensors of ONE type and one row length; otherwise every K-quant member is uploaded on its own
// (the reference sends such layers through its Q8 re-quantisation, which is not part of this library).
// Members that are absent or not K-quant stay empty (w == NULL, qtype = the file's type or -1).
int bpq4k_gguf_load_layer(bpq4k_handle_t h, bpq4k_gguf_t g, uint32_t layer, int q6_layout, bpq4k_layer_weights* out) {
    if (!h || !g || !out) return BPQ4K_ERR_INVALID_ARG;
    std::memset(out, 0, sizeof(*out));
    const std::string pfx = "blk." + std::to_string(layer) + ".";
    auto find = [&](const char* name, uint64_t* idx) {
        auto it = g->index.find(pfx + name);
        if (it == g->index.end()) return false;
        *idx = it->second;
        return true;
    };
    auto type_of = [&](uint64_t idx) { return g->tensors[(size_t)idx].type; };
    auto put = [&](bpq4k_kq_tensor* dst, const uint64_t* idx, uint32_t n) -> int {
        const int layout = (type_of(idx[0]) == BPQ4K_TYPE_Q6_K && q6_layout == BPQ4K_TYPE_Q6_K_PADDED) ? BPQ4K_TYPE_Q6_K_PADDED : 0;
        dst->n_fused = n;
        return bpq4k_gguf_upload_fused(h, g, idx, n, layout, &dst->w, &dst->qtype, &dst->N, &dst->K, &dst->rowStrideWords);
    };
    auto single = [&](const char* name, bpq4k_kq_tensor* dst) -> int {
        uint64_t idx;
        dst->qtype = -1;
        if (!find(name, &idx)) return BPQ4K_OK;
        dst->qtype = (int)type_of(idx);
        if (!is_kquant(type_of(idx))) return BPQ4K_OK;
        return put(dst, &idx, 1);
    };
    auto same_rows = [&](const uint64_t* idx, uint32_t n) {
        for (uint32_t i = 0; i < n; i++)
            if (!is_kquant(type_of(idx[i])) || type_of(idx[i]) != type_of(idx[0]) ||
                g->tensors[(size_t)idx[i]].shape[0] != g->tensors[(size_t)idx[0]].shape[0])
                return false;
        return true;
    };
    int st = BPQ4K_OK;
    uint64_t q, k, v, qkv, gi, ui;
    out->qkv.qtype = out->q.qtype = out->k.qtype = out->v.qtype = -1;
    out->gate_up.qtype = out->gate.qtype = out->up.qtype = -1;
    const bool hq = find("attn_q.weight", &q), hk = find("attn_k.weight", &k), hv = find("attn_v.weight", &v);
    if (!hq && find("attn_qkv.weight", &qkv)) {
        out->qkv.qtype = (int)type_of(qkv);
        if (is_kquant(type_of(qkv))) st = put(&out->qkv, &qkv, 1);
        out->qkv_prefused = 1;
    } else if (hq && hk && hv) {
        const uint64_t idx[3] = {q, k, v};
        if (same_rows(idx, 3)) {
            st = put(&out->qkv, idx, 3);
        } else {
            st = single("attn_q.weight", &out->q);
            if (st == BPQ4K_OK) st = single("attn_k.weight", &out->k);
            if (st == BPQ4K_OK) st = single("attn_v.weight", &out->v);
        }
    } else if (hq) {  // layers that share K/V with an earlier layer ship attn_q only
        st = single("attn_q.weight", &out->q);
    }
    if (st == BPQ4K_OK) st = single("attn_output.weight", &out->o);
    if (st == BPQ4K_OK) {
        if (find("ffn_gate.weight", &gi) && find("ffn_up.weight", &ui)) {
            const uint64_t idx[2] = {gi, ui};
            if (same_rows(idx, 2)) {
                st = put(&out->gate_up, idx, 2);
            } else {
                st = single("ffn_gate.weight", &out->gate);
                if (st == BPQ4K_OK) st = single("ffn_up.weight", &out->up);
            }
        }
    }
    if (st == BPQ4K_OK) st = single("ffn_down.weight", &out->down);
    if (st != BPQ4K_OK) bpq4k_free_layer(h, out);
    return st;
}

int bpq4k_free_layer(bpq4k_handle_t h, bpq4k_layer_weights* lw) {
    if (!h || !lw) return BPQ4K_ERR_INVALID_ARG;
    for (bpq4k_kq_tensor* t : {&lw->qkv, &lw->q, &lw->k, &lw->v, &lw->o, &lw->gate_up, &lw->gate, &lw->up, &lw->down}) {
        if (t->w) bpq4k_free_device(h, t->w);
        t->w = nullptr;
    }
    return BPQ4K_OK;
}

}  // extern "C"
#pragma GCC visibility pop
