// bpq4k_op_test_runner -- the reference's op_test_runner harness (runtime/op_test_runner.cpp)
// on top of the CUDA-backed interface: same command line, same files, same strings.
//
//   bpq4k_op_test_runner <model.onnx> <input_dir> <output_dir>
//
//   <input_dir>/manifest.json   {"inputs": [{"name": ..., "dtype": ..., "shape": [...]}, ...]}
//   <input_dir>/<name>.bin      raw little-endian bytes; a missing file means zeros
//   <output_dir>/<name>.bin and <output_dir>/manifest.json ({"outputs": [...]})
//   dtype strings: float32 float16 int32 int64 uint8 bool (int8 on output only)
//   stderr "Execute: %.1fms"; stdout "OK"; exit status 0, or 1 on any setup failure.
//
// `--parse-only` (an extra first argument) loads the model and the manifest and prints the
// graph without touching a device; it lets the file handling be tested on machines with no GPU.
#include <chrono>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <string>
#include <vector>

#include "bp_runtime.h"
#include "json_min.h"

namespace fs = std::filesystem;

static TensorDtype parseDtype(const std::string& s) {
    if (s == "float16") return TensorDtype::Float16;
    if (s == "int32") return TensorDtype::Int32;
    if (s == "int64") return TensorDtype::Int64;
    if (s == "uint8") return TensorDtype::UInt8;
    if (s == "bool") return TensorDtype::Bool;
    return TensorDtype::Float32;  // "float32" and anything unknown, like the reference
}

static const char* dtypeStr(TensorDtype d) {
    switch (d) {
        case TensorDtype::Float16: return "float16";
        case TensorDtype::Int32: return "int32";
        case TensorDtype::Int64: return "int64";
        case TensorDtype::UInt8: return "uint8";
        case TensorDtype::Int8: return "int8";
        case TensorDtype::Bool: return "bool";
        default: return "float32";
    }
}

struct InputSpec {
    std::string name;
    TensorDtype dtype;
    std::vector<int64_t> shape;
};

static bool readManifest(const std::string& dir, std::vector<InputSpec>& specs) {
    const std::string path = (fs::path(dir) / "manifest.json").string();
    std::ifstream mf(path);
    if (!mf.is_open()) {
        fprintf(stderr, "Cannot open: %s\n", path.c_str());
        return false;
    }
    const std::string text{std::istreambuf_iterator<char>(mf), std::istreambuf_iterator<char>()};
    jsonmin::Value root;
    if (!jsonmin::parse(text, root)) {
        fprintf(stderr, "Cannot parse: %s\n", path.c_str());
        return false;
    }
    const jsonmin::Value& arr = root["inputs"];
    for (size_t i = 0; i < arr.size(); i++) {
        InputSpec s;
        s.name = arr[i]["name"].str;
        s.dtype = parseDtype(arr[i]["dtype"].str);
        const jsonmin::Value& sh = arr[i]["shape"];
        for (size_t j = 0; j < sh.size(); j++) s.shape.push_back((int64_t)sh[j].num);
        specs.push_back(std::move(s));
    }
    return true;
}

int main(int argc, char* argv[]) {
    bool parseOnly = false;
    int a0 = 1;
    if (argc > 1 && std::strcmp(argv[1], "--parse-only") == 0) {
        parseOnly = true;
        a0 = 2;
    }
    if (argc - a0 < 3) {
        fprintf(stderr, "Usage: %s <model.onnx> <input_dir> <output_dir>\n", argv[0]);
        return 1;
    }
    const std::string modelPath = argv[a0], inputDir = argv[a0 + 1], outputDir = argv[a0 + 2];
    fs::create_directories(outputDir);

    if (parseOnly) {
        std::ifstream f(modelPath, std::ios::binary);
        if (!f.is_open()) {
            fprintf(stderr, "Failed to load: %s\n", modelPath.c_str());
            return 1;
        }
        std::vector<uint8_t> bytes((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
        OnnxGraph g;
        std::string err;
        if (!ParseOnnxModel(bytes.data(), bytes.size(), g, &err)) {
            fprintf(stderr, "Failed to load: %s (%s)\n", modelPath.c_str(), err.c_str());
            return 1;
        }
        std::vector<InputSpec> specs;
        if (!readManifest(inputDir, specs)) return 1;
        for (auto& n : g.nodes) {
            printf("node %s op=%s registered=%d inputs=%zu outputs=%zu", n.name.c_str(), n.opType.c_str(),
                   (int)GraphExecutor::GetOpRegistry().count(n.opType), n.inputs.size(), n.outputs.size());
            for (auto& kv : n.attrInts) printf(" %s=%lld", kv.first.c_str(), (long long)kv.second);
            printf("\n");
        }
        for (auto& kv : g.initializers) printf("initializer %s dtype=%s bytes=%zu\n", kv.first.c_str(), dtypeStr(kv.second.dtype), kv.second.data.size());
        for (auto& v : g.inputs) printf("graph-input %s dtype=%s rank=%zu\n", v.name.c_str(), dtypeStr(v.dtype), v.shape.size());
        for (auto& v : g.outputs) printf("graph-output %s dtype=%s rank=%zu\n", v.name.c_str(), dtypeStr(v.dtype), v.shape.size());
        for (auto& s : specs) printf("manifest-input %s dtype=%s rank=%zu\n", s.name.c_str(), dtypeStr(s.dtype), s.shape.size());
        printf("OK\n");
        return 0;
    }

    // 1. device
    GPUContext gpu;
    if (!gpu.init(0)) {
        fprintf(stderr, "Failed to init GPU\n");
        return 1;
    }
    // 2. model
    GraphExecutor executor;
    if (!executor.Load(gpu, modelPath)) {
        fprintf(stderr, "Failed to load: %s\n", modelPath.c_str());
        return 1;
    }
    // 3. manifest
    std::vector<InputSpec> specs;
    if (!readManifest(inputDir, specs)) return 1;
    // 4. inputs
    std::unordered_map<std::string, GpuTensor> inputTensors;
    std::unordered_map<std::string, GpuTensor*> inputs;
    for (auto& s : specs) {
        const std::string binPath = (fs::path(inputDir) / (s.name + ".bin")).string();
        std::vector<uint8_t> data;
        std::ifstream bin(binPath, std::ios::binary);
        if (!bin.is_open()) {
            fprintf(stderr, "Cannot open input: %s\n", binPath.c_str());
            int64_t nel = 1;
            for (auto d : s.shape) nel *= d;
            data.assign((size_t)nel * GpuTensor::DtypeSizeOf(s.dtype), 0);  // zeros, as the reference does
        } else {
            data.assign(std::istreambuf_iterator<char>(bin), std::istreambuf_iterator<char>());
        }
        GpuTensor& t = inputTensors[s.name];
        t.shape = s.shape;
        t.dtype = s.dtype;
        t.buffer = gpu.createBuffer(s.name, data.empty() ? 4 : data.size());
        if (!data.empty()) gpu.writeBuffer(t.buffer, data.data(), data.size());
        t.cpuData = std::move(data);
        inputs[s.name] = &t;
    }
    // 5. output placeholders
    std::unordered_map<std::string, GpuTensor> outputTensors;
    std::unordered_map<std::string, GpuTensor*> outputs;
    std::vector<std::string> outputNames;
    for (auto& o : executor.GetGraph().outputs) {
        outputNames.push_back(o.name);
        GpuTensor& t = outputTensors[o.name];
        t.shape = o.shape;
        t.dtype = o.dtype;
        outputs[o.name] = &t;  // filled by Execute when the producing op succeeded
    }
    // 6. run
    const auto t0 = std::chrono::steady_clock::now();
    executor.Execute(inputs, outputs);
    executor.FlushPendingWork();
    gpu.waitForQueue();
    const auto t1 = std::chrono::steady_clock::now();
    fprintf(stderr, "Execute: %.1fms\n", std::chrono::duration<double, std::milli>(t1 - t0).count());
    // 7. outputs
    std::string manifest = "{\n  \"outputs\": [\n";
    bool first = true;
    for (auto& name : outputNames) {
        GpuTensor* t = outputs[name];
        if (!t || !t->buffer.handle) {
            fprintf(stderr, "Output '%s' not valid\n", name.c_str());
            continue;
        }
        const size_t bytes = t->ByteSize() ? t->ByteSize() : 4;
        const std::vector<uint8_t> data = gpu.readBuffer(t->buffer, bytes);
        std::ofstream bin((fs::path(outputDir) / (name + ".bin")).string(), std::ios::binary);
        if (bin.is_open()) bin.write(reinterpret_cast<const char*>(data.data()), (std::streamsize)data.size());
        if (!first) manifest += ",\n";
        first = false;
        manifest += "    {\"name\": \"" + name + "\", \"dtype\": \"" + dtypeStr(t->dtype) + "\", \"shape\": [";
        for (size_t j = 0; j < t->shape.size(); j++) manifest += (j ? ", " : "") + std::to_string(t->shape[j]);
        manifest += "]}";
    }
    manifest += "\n  ]\n}\n";
    std::ofstream omf((fs::path(outputDir) / "manifest.json").string());
    omf << manifest;
    omf.close();
    if (gpu.deviceLost) {
        fprintf(stderr, "device reported an error\n");
        return 1;
    }
    printf("OK\n");
    return 0;
}
