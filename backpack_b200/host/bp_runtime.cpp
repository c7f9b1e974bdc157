// CUDA-backed implementation of the interface in bp_runtime.h, including a small
// protobuf reader for the ONNX subset (wire format only; no protobuf library).
#include "bp_runtime.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <fstream>

// ---------------------------------------------------------------- GPUContext

GPUContext::~GPUContext() {
    if (device_ < 0) return;
    cudaSetDevice(device_);
    if (q4k_) bpq4k_destroy(q4k_);
    for (void* p : owned_) cudaFree(p);
    if (stream_) cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
}

bool GPUContext::init(int device) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device >= count) {
        cudaGetLastError();
        return false;
    }
    if (cudaSetDevice(device) != cudaSuccess) return false;
    cudaStream_t s;
    if (cudaStreamCreate(&s) != cudaSuccess) return false;
    stream_ = s;
    device_ = device;
    const int st = bpq4k_create(device, &q4k_);
    if (st != BPQ4K_OK) {
        fprintf(stderr, "bpq4k_create failed: %s\n", bpq4k_status_string(st));
        return false;
    }
    return true;
}

GPUBuffer GPUContext::createBuffer(const std::string& name, uint64_t bytes) {
    (void)name;
    GPUBuffer b;
    if (bytes == 0) bytes = 4;
    // 256-byte granularity keeps every buffer 16-byte aligned with room for vector loads
    const uint64_t alloc = (bytes + 255) / 256 * 256;
    void* p = nullptr;
    if (cudaMalloc(&p, alloc) != cudaSuccess) {
        cudaGetLastError();
        lastAllocFailed = true;
        fprintf(stderr, "[gpu] allocation of %llu bytes failed\n", (unsigned long long)alloc);
        return b;
    }
    cudaMemsetAsync(p, 0, alloc, static_cast<cudaStream_t>(stream_));
    owned_.push_back(p);
    b.handle = p;
    b.size = bytes;
    return b;
}

void GPUContext::releaseBuffer(GPUBuffer& b) {
    for (auto& p : owned_)
        if (p == b.handle) {
            cudaFree(p);
            p = owned_.back();
            owned_.pop_back();
            break;
        }
    b = GPUBuffer{};
}

void GPUContext::writeBuffer(const GPUBuffer& b, const void* data, uint64_t bytes, uint64_t offset) {
    if (!b.handle || !bytes) return;
    if (cudaMemcpyAsync(static_cast<uint8_t*>(b.handle) + offset, data, bytes, cudaMemcpyHostToDevice,
                        static_cast<cudaStream_t>(stream_)) != cudaSuccess)
        deviceLost = true;
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));  // the caller may free `data` right away
}

std::vector<uint8_t> GPUContext::readBuffer(const GPUBuffer& b, uint64_t bytes) {
    std::vector<uint8_t> out(bytes);
    if (!b.handle || !bytes) return out;
    cudaStream_t s = static_cast<cudaStream_t>(stream_);
    if (cudaMemcpyAsync(out.data(), b.handle, bytes, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        fprintf(stderr, "[gpu] read-back failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        deviceLost = true;
    }
    return out;
}

void GPUContext::waitForQueue() {
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)) != cudaSuccess) {
        fprintf(stderr, "[gpu] queue wait failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        deviceLost = true;
    }
    int st = 0;
    if (q4k_ && bpq4k_device_status(q4k_, stream_, &st) != BPQ4K_OK) {
        fprintf(stderr, "[gpu] %s\n", bpq4k_last_error_string(q4k_));
        deviceLost = true;
    }
}

// ---------------------------------------------------------------- OpContext

GpuTensor OpContext::AllocTensor(std::vector<int64_t> shape, TensorDtype dtype) { return ex_.AllocTensor(std::move(shape), dtype); }
void OpContext::EnsureGpu(GpuTensor& t) { ex_.EnsureGpu(t); }
GPUContext* OpContext::getGpu() { return ex_.gpu; }

// ---------------------------------------------------------------- GraphExecutor

std::unordered_map<std::string, OpDispatchFn>& GraphExecutor::GetOpRegistry() {
    static std::unordered_map<std::string, OpDispatchFn> registry;  // filled during static initialisation
    return registry;
}

void GraphExecutor::RegisterOp(const std::string& opType, OpDispatchFn fn) { GetOpRegistry()[opType] = std::move(fn); }

GpuTensor GraphExecutor::AllocTensor(std::vector<int64_t> shape, TensorDtype dtype) {
    GpuTensor t;
    t.shape = std::move(shape);
    t.dtype = dtype;
    t.buffer = gpu->createBuffer("tensor", t.ByteSize());
    return t;
}

void GraphExecutor::EnsureGpu(GpuTensor& t) {
    if (t.buffer.handle || t.cpuData.empty()) return;
    t.buffer = gpu->createBuffer("upload", t.cpuData.size());
    gpu->writeBuffer(t.buffer, t.cpuData.data(), t.cpuData.size());
    t.isCpuOnly = false;
}

bool GraphExecutor::Load(GPUContext& gpuCtx, const std::string& onnxPath) {
    std::ifstream f(onnxPath, std::ios::binary);
    if (!f.is_open()) {
        fprintf(stderr, "Cannot open model: %s\n", onnxPath.c_str());
        return false;
    }
    std::vector<uint8_t> bytes((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    return LoadFromMemory(gpuCtx, bytes.data(), bytes.size());
}

bool GraphExecutor::LoadFromMemory(GPUContext& gpuCtx, const uint8_t* data, size_t size) {
    gpu = &gpuCtx;
    std::string err;
    if (!ParseOnnxModel(data, size, graph_, &err)) {
        fprintf(stderr, "ONNX parse error: %s\n", err.c_str());
        return false;
    }
    for (auto& kv : graph_.initializers) {  // weights are uploaded once, at load
        GpuTensor t;
        t.shape = kv.second.shape;
        t.dtype = kv.second.dtype;
        t.cpuData = kv.second.data;
        EnsureGpu(t);
        weightStore_[kv.first] = std::move(t);
    }
    return true;
}

void GraphExecutor::Execute(const std::unordered_map<std::string, GpuTensor*>& inputs,
                            std::unordered_map<std::string, GpuTensor*>& outputs) {
    tensorStore_.clear();
    auto find = [&](const std::string& name) -> GpuTensor* {
        if (name.empty()) return nullptr;
        auto i = inputs.find(name);
        if (i != inputs.end()) return i->second;
        auto w = weightStore_.find(name);
        if (w != weightStore_.end()) return &w->second;
        auto t = tensorStore_.find(name);
        if (t != tensorStore_.end()) return &t->second;
        return nullptr;
    };
    OpContext ctx(*this);
    auto& registry = GetOpRegistry();
    for (const auto& node : graph_.nodes) {  // ONNX stores nodes in topological order
        auto op = registry.find(node.opType);
        if (op == registry.end()) {
            fprintf(stderr, "[exec] no implementation for op '%s' (node '%s')\n", node.opType.c_str(), node.name.c_str());
            continue;
        }
        std::vector<GpuTensor*> in, out;
        for (const auto& n : node.inputs) in.push_back(find(n));
        for (const auto& n : node.outputs) out.push_back(&tensorStore_[n]);
        op->second(ctx, node, in, out);
    }
    for (auto& kv : outputs) {
        auto t = tensorStore_.find(kv.first);
        if (t != tensorStore_.end() && t->second.IsValid()) *kv.second = t->second;
    }
}

void GraphExecutor::FlushPendingWork() {}  // ops enqueue directly on the context's stream

// ---------------------------------------------------------------- ONNX wire format

namespace {

struct Reader {
    const uint8_t* p;
    const uint8_t* end;
    bool ok = true;
    bool done() const { return p >= end || !ok; }
    uint64_t varint() {
        uint64_t v = 0;
        int shift = 0;
        while (p < end && shift < 64) {
            const uint8_t b = *p++;
            v |= (uint64_t)(b & 0x7F) << shift;
            if (!(b & 0x80)) return v;
            shift += 7;
        }
        ok = false;
        return 0;
    }
    Reader sub() {
        const uint64_t n = varint();
        if (!ok || n > (uint64_t)(end - p)) {
            ok = false;
            return Reader{p, p, false};
        }
        Reader r{p, p + n};
        p += n;
        return r;
    }
    void skip(uint32_t wire) {
        switch (wire) {
            case 0: varint(); break;
            case 1: p += 8; break;
            case 2: sub(); break;
            case 5: p += 4; break;
            default: ok = false;
        }
        if (p > end) ok = false;
    }
    std::string str() {
        Reader r = sub();
        return std::string(reinterpret_cast<const char*>(r.p), (size_t)(r.end - r.p));
    }
};

bool dtype_from_onnx(int64_t code, TensorDtype& out) {
    switch (code) {
        case 1: out = TensorDtype::Float32; return true;
        case 2: out = TensorDtype::UInt8; return true;
        case 3: out = TensorDtype::Int8; return true;
        case 6: out = TensorDtype::Int32; return true;
        case 7: out = TensorDtype::Int64; return true;
        case 9: out = TensorDtype::Bool; return true;
        case 10: out = TensorDtype::Float16; return true;
        default: return false;
    }
}

void parse_tensor(Reader r, std::string& name, OnnxInitData& t) {
    std::vector<float> floats;
    std::vector<int64_t> ints;
    int64_t code = 1;
    while (!r.done()) {
        const uint64_t key = r.varint();
        const uint32_t field = (uint32_t)(key >> 3), wire = (uint32_t)(key & 7);
        if (field == 1 && wire == 0) t.shape.push_back((int64_t)r.varint());
        else if (field == 1 && wire == 2) { Reader s = r.sub(); while (!s.done()) t.shape.push_back((int64_t)s.varint()); }
        else if (field == 2 && wire == 0) code = (int64_t)r.varint();
        else if (field == 8 && wire == 2) name = r.str();
        else if (field == 9 && wire == 2) { Reader s = r.sub(); t.data.assign(s.p, s.end); }
        else if (field == 4 && wire == 2) { Reader s = r.sub(); floats.resize((size_t)(s.end - s.p) / 4); memcpy(floats.data(), s.p, floats.size() * 4); }
        else if (field == 4 && wire == 5) { float v; memcpy(&v, r.p, 4); r.p += 4; floats.push_back(v); }
        else if ((field == 5 || field == 7) && wire == 2) { Reader s = r.sub(); while (!s.done()) ints.push_back((int64_t)s.varint()); }
        else if ((field == 5 || field == 7) && wire == 0) ints.push_back((int64_t)r.varint());
        else r.skip(wire);
    }
    dtype_from_onnx(code, t.dtype);
    if (t.data.empty() && !floats.empty()) {
        t.data.resize(floats.size() * 4);
        memcpy(t.data.data(), floats.data(), t.data.size());
    } else if (t.data.empty() && !ints.empty()) {
        const size_t es = GpuTensor::DtypeSizeOf(t.dtype);
        t.data.resize(ints.size() * es);
        for (size_t i = 0; i < ints.size(); i++) memcpy(t.data.data() + i * es, &ints[i], es);  // little-endian truncation
    }
}

void parse_value_info(Reader r, OnnxGraphInput& v) {
    while (!r.done()) {
        const uint64_t key = r.varint();
        const uint32_t field = (uint32_t)(key >> 3), wire = (uint32_t)(key & 7);
        if (field == 1 && wire == 2) v.name = r.str();
        else if (field == 2 && wire == 2) {  // TypeProto
            Reader tp = r.sub();
            while (!tp.done()) {
                const uint64_t k2 = tp.varint();
                if ((k2 >> 3) == 1 && (k2 & 7) == 2) {  // tensor_type
                    Reader tt = tp.sub();
                    while (!tt.done()) {
                        const uint64_t k3 = tt.varint();
                        if ((k3 >> 3) == 1 && (k3 & 7) == 0) dtype_from_onnx((int64_t)tt.varint(), v.dtype);
                        else if ((k3 >> 3) == 2 && (k3 & 7) == 2) {  // TensorShapeProto
                            Reader sh = tt.sub();
                            while (!sh.done()) {
                                const uint64_t k4 = sh.varint();
                                if ((k4 >> 3) == 1 && (k4 & 7) == 2) {  // Dimension
                                    Reader dm = sh.sub();
                                    int64_t val = -1;
                                    while (!dm.done()) {
                                        const uint64_t k5 = dm.varint();
                                        if ((k5 >> 3) == 1 && (k5 & 7) == 0) val = (int64_t)dm.varint();
                                        else dm.skip((uint32_t)(k5 & 7));
                                    }
                                    v.shape.push_back(val);
                                } else sh.skip((uint32_t)(k4 & 7));
                            }
                        } else tt.skip((uint32_t)(k3 & 7));
                    }
                } else tp.skip((uint32_t)(k2 & 7));
            }
        } else r.skip(wire);
    }
}

void parse_attribute(Reader r, OnnxGraphNode& n) {
    std::string name, s;
    int64_t i = 0;
    float f = 0;
    bool has_i = false, has_f = false, has_s = false;
    std::vector<int64_t> ints;
    while (!r.done()) {
        const uint64_t key = r.varint();
        const uint32_t field = (uint32_t)(key >> 3), wire = (uint32_t)(key & 7);
        if (field == 1 && wire == 2) name = r.str();
        else if (field == 2 && wire == 5) { memcpy(&f, r.p, 4); r.p += 4; has_f = true; }
        else if (field == 3 && wire == 0) { i = (int64_t)r.varint(); has_i = true; }
        else if (field == 4 && wire == 2) { s = r.str(); has_s = true; }
        else if (field == 8 && wire == 2) { Reader q = r.sub(); while (!q.done()) ints.push_back((int64_t)q.varint()); }
        else if (field == 8 && wire == 0) ints.push_back((int64_t)r.varint());
        else r.skip(wire);
    }
    if (has_i) n.attrInts[name] = i;
    if (has_f) n.attrFloats[name] = f;
    if (has_s) n.attrStrings[name] = s;
    if (!ints.empty()) n.attrIntLists[name] = ints;
}

void parse_node(Reader r, OnnxGraphNode& n) {
    while (!r.done()) {
        const uint64_t key = r.varint();
        const uint32_t field = (uint32_t)(key >> 3), wire = (uint32_t)(key & 7);
        if (wire != 2) { r.skip(wire); continue; }
        switch (field) {
            case 1: n.inputs.push_back(r.str()); break;
            case 2: n.outputs.push_back(r.str()); break;
            case 3: n.name = r.str(); break;
            case 4: n.opType = r.str(); break;
            case 5: parse_attribute(r.sub(), n); break;
            case 7: n.domain = r.str(); break;
            default: r.skip(wire);
        }
    }
}

void parse_graph(Reader r, OnnxGraph& g) {
    while (!r.done()) {
        const uint64_t key = r.varint();
        const uint32_t field = (uint32_t)(key >> 3), wire = (uint32_t)(key & 7);
        if (wire != 2) { r.skip(wire); continue; }
        switch (field) {
            case 1: { OnnxGraphNode n; parse_node(r.sub(), n); g.nodes.push_back(std::move(n)); break; }
            case 5: { std::string name; OnnxInitData t; parse_tensor(r.sub(), name, t); g.initializers[name] = std::move(t); break; }
            case 11: { OnnxGraphInput v; parse_value_info(r.sub(), v); g.inputs.push_back(std::move(v)); break; }
            case 12: { OnnxGraphInput v; parse_value_info(r.sub(), v); g.outputs.push_back(std::move(v)); break; }
            default: r.skip(wire);
        }
    }
    // graph inputs that are initializers are weights, not runtime inputs
    std::vector<OnnxGraphInput> real;
    for (auto& v : g.inputs)
        if (!g.initializers.count(v.name)) real.push_back(v);
    g.inputs.swap(real);
}

}  // namespace

bool ParseOnnxModel(const uint8_t* data, size_t size, OnnxGraph& out, std::string* error) {
    out = OnnxGraph{};
    Reader r{data, data + size};
    bool saw_graph = false;
    while (!r.done()) {
        const uint64_t key = r.varint();
        const uint32_t field = (uint32_t)(key >> 3), wire = (uint32_t)(key & 7);
        if (field == 7 && wire == 2) {
            Reader g = r.sub();
            if (!r.ok) break;
            parse_graph(g, out);
            saw_graph = true;
        } else r.skip(wire);
    }
    if (!r.ok || !saw_graph) {
        if (error) *error = !r.ok ? "malformed protobuf" : "no graph in model";
        return false;
    }
    return true;
}
