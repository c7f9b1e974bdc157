// Host-side mirror of the Backpack runtime's operator interface for the one
// operator this library provides, backed by CUDA device buffers instead of
// Dawn/WebGPU buffers.
//
// The shapes follow the reference so that an op written against it reads the
// same here: GPUBuffer / GPUContext (runtime/gpu_context.h:36-44,151-220),
// TensorDtype / GpuTensor (runtime/graph_executor.h:30-66), OnnxGraphNode with
// GetInt/GetFloat (:70-90), OnnxGraph (:94-115), OpDispatchFn (:149-153),
// GraphExecutor::Load / Execute / GetGraph / RegisterOp / GetOpRegistry
// (:159-254, runtime/graph_executor.cpp:209-216) and REGISTER_OP (:374-377).
// Everything that exists only to serve WGSL (pipelines, bind groups, shader
// templating, fusion, capture/replay) has no counterpart.
#pragma once
#include <cstdint>
#include <functional>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/bpq4k.h"

struct GPUBuffer {
    void* handle = nullptr;  // device pointer
    uint64_t size = 0;
};

// One CUDA device + one stream + one bpq4k handle.  Stands in for the Dawn
// device/queue wrapper; single-threaded like the original.
class GPUContext {
public:
    ~GPUContext();
    bool init(int device = 0);
    GPUBuffer createBuffer(const std::string& name, uint64_t bytes);
    void releaseBuffer(GPUBuffer& b);
    void writeBuffer(const GPUBuffer& b, const void* data, uint64_t bytes, uint64_t offset = 0);
    std::vector<uint8_t> readBuffer(const GPUBuffer& b, uint64_t bytes);
    void waitForQueue();
    bpq4k_handle_t q4k() const { return q4k_; }
    void* stream() const { return stream_; }
    bool deviceLost = false;       // set when a CUDA call or a kernel reports failure
    bool lastAllocFailed = false;  // set when createBuffer could not allocate

private:
    int device_ = -1;
    void* stream_ = nullptr;
    bpq4k_handle_t q4k_ = nullptr;
    std::vector<void*> owned_;
};

enum class TensorDtype { Float32, Float16, Int32, Int64, UInt8, Int8, Bool };

struct GpuTensor {
    GPUBuffer buffer;
    std::vector<int64_t> shape;
    TensorDtype dtype = TensorDtype::Float32;
    std::vector<uint8_t> cpuData;  // small metadata tensors / initializers before upload
    bool isCpuOnly = false;

    int64_t ElementCount() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
    static size_t DtypeSizeOf(TensorDtype dt) {
        switch (dt) {
            case TensorDtype::Float32: case TensorDtype::Int32: return 4;
            case TensorDtype::Float16: return 2;
            case TensorDtype::Int64: return 8;
            default: return 1;
        }
    }
    size_t DtypeSize() const { return DtypeSizeOf(dtype); }
    size_t ByteSize() const { return (size_t)ElementCount() * DtypeSize(); }
    bool IsValid() const { return buffer.handle != nullptr || isCpuOnly; }
};

struct OnnxGraphNode {
    std::string opType, name, domain;
    std::vector<std::string> inputs, outputs;
    std::unordered_map<std::string, int64_t> attrInts;
    std::unordered_map<std::string, float> attrFloats;
    std::unordered_map<std::string, std::string> attrStrings;
    std::unordered_map<std::string, std::vector<int64_t>> attrIntLists;
    int64_t GetInt(const std::string& key, int64_t def = 0) const {
        auto it = attrInts.find(key);
        return it != attrInts.end() ? it->second : def;
    }
    float GetFloat(const std::string& key, float def = 0.0f) const {
        auto it = attrFloats.find(key);
        return it != attrFloats.end() ? it->second : def;
    }
};

struct OnnxGraphInput {
    std::string name;
    TensorDtype dtype = TensorDtype::Float32;
    std::vector<int64_t> shape;  // -1 for dynamic dims
};

struct OnnxInitData {
    std::vector<uint8_t> data;
    TensorDtype dtype = TensorDtype::Float32;
    std::vector<int64_t> shape;
};

struct OnnxGraph {
    std::vector<OnnxGraphNode> nodes;
    std::vector<OnnxGraphInput> inputs, outputs;
    std::unordered_map<std::string, OnnxInitData> initializers;
};

class GraphExecutor;

// What an op sees: allocation and upload helpers plus the device context.
class OpContext {
public:
    explicit OpContext(GraphExecutor& ex) : ex_(ex) {}
    GpuTensor AllocTensor(std::vector<int64_t> shape, TensorDtype dtype);
    void EnsureGpu(GpuTensor& t);
    GPUContext* getGpu();

private:
    GraphExecutor& ex_;
};

using OpDispatchFn = std::function<void(OpContext& ctx, const OnnxGraphNode& node,
                                        const std::vector<GpuTensor*>& inputs, std::vector<GpuTensor*>& outputs)>;

class GraphExecutor {
public:
    GPUContext* gpu = nullptr;

    bool Load(GPUContext& gpuCtx, const std::string& onnxPath);
    bool LoadFromMemory(GPUContext& gpuCtx, const uint8_t* data, size_t size);
    void Execute(const std::unordered_map<std::string, GpuTensor*>& inputs,
                 std::unordered_map<std::string, GpuTensor*>& outputs);
    void FlushPendingWork();
    const OnnxGraph& GetGraph() const { return graph_; }
    GpuTensor AllocTensor(std::vector<int64_t> shape, TensorDtype dtype);
    void EnsureGpu(GpuTensor& t);

    static void RegisterOp(const std::string& opType, OpDispatchFn fn);
    static std::unordered_map<std::string, OpDispatchFn>& GetOpRegistry();

private:
    OnnxGraph graph_;
    std::unordered_map<std::string, GpuTensor> weightStore_;  // initializers, uploaded at Load
    std::unordered_map<std::string, GpuTensor> tensorStore_;  // intermediates of the last Execute
};

#define REGISTER_OP(name, fn)                                             \
    static struct _RegOp_##name {                                         \
        _RegOp_##name() { GraphExecutor::RegisterOp(#name, fn); }         \
    } _regOp_##name;

// Parse the subset of ONNX the reference's loader needs (ModelProto.graph;
// GraphProto node/initializer/input/output; NodeProto input/output/name/op_type/
// attribute/domain; AttributeProto name/f/i/s/ints; TensorProto dims/data_type/
// raw_data/name and the typed repeated fields; ValueInfoProto tensor types).
bool ParseOnnxModel(const uint8_t* data, size_t size, OnnxGraph& out, std::string* error);
