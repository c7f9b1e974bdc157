// ref_shim.cpp -- C-callable doorway into the reference's own CPU code for the
// Q4_K path (and its Q5_K / Q6_K siblings), so the restatement in q4k_oracle.c can be checked against it and
// so the benchmark can time the reference itself on the host cores.
//
// TEST INFRASTRUCTURE ONLY.  This file contains no reference code: it includes
// the reference's header and is linked with the reference's gguf_loader.cpp,
// both compiled where they lie in the mounted reference tree (see the Makefile
// target `ref`).  The result goes to oracle/_ref/, which is not committed.
#include "gguf_loader.h"   // -I <reference>/runtime

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

extern "C" {

// dequant_kquant(..., GGUF_TYPE_Q4_K) -- runtime/gguf_loader.cpp:455-496
void ref_q4k_dequant(const void* raw, float* out, uint32_t N, uint32_t K) {
    dequant_kquant(raw, out, N, K, GGUF_TYPE_Q4_K);
}

// pack_q4k -- runtime/gguf_loader.cpp:359-379.  Copies the packed words out and
// reports the two derived fields of KQuantPacked.
void ref_pack_q4k(const void* raw, uint32_t N, uint32_t K, uint32_t* words,
                  uint32_t* rowStrideWords, uint32_t* nBlocks) {
    KQuantPacked p = pack_q4k(raw, N, K);
    if (rowStrideWords) *rowStrideWords = p.rowStrideWords;
    if (nBlocks) *nBlocks = p.nBlocks;
    if (words) std::memcpy(words, p.data.data(), p.data.size() * sizeof(uint32_t));
}

// The expected-value computation of runtime/tests/kernel_test.cpp:1682,1688,
// 1728,1746: dequant_kquant, then for each (m, n) a float accumulator that
// starts at bias[n] and adds x*w for k ascending.  The tests decode the whole
// matrix first; here rows are decoded in slabs of 64 with the same reference
// routine so the scratch stays cache-sized (the arithmetic per output is the
// same sequence of float operations).
static void rows(const float* X, const uint8_t* raw, const float* bias, float* Y,
                 uint32_t M, uint32_t N, uint32_t K, uint32_t n0, uint32_t n1) {
    const uint32_t nb = K / 256, SLAB = 64;
    std::vector<float> deq((size_t)SLAB * K);
    for (uint32_t s0 = n0; s0 < n1; s0 += SLAB) {
        const uint32_t cnt = (n1 - s0 < SLAB) ? n1 - s0 : SLAB;
        dequant_kquant(raw + (size_t)s0 * nb * 144, deq.data(), cnt, K, GGUF_TYPE_Q4_K);
        for (uint32_t m = 0; m < M; m++)
            for (uint32_t r = 0; r < cnt; r++) {
                const uint32_t n = s0 + r;
                float a = bias ? bias[n] : 0.0f;
                for (uint32_t k = 0; k < K; k++) a += X[(size_t)m * K + k] * deq[(size_t)r * K + k];
                Y[(size_t)m * N + n] = a;
            }
    }
}

void ref_q4k_matmul(const float* X, const void* raw, const float* bias, float* Y,
                    uint32_t M, uint32_t N, uint32_t K, uint32_t threads) {
    const uint8_t* src = (const uint8_t*)raw;
    if (threads <= 1 || N < threads) {
        rows(X, src, bias, Y, M, N, K, 0, N);
        return;
    }
    // Row-parallel: each thread decodes and multiplies its own contiguous rows.
    std::vector<std::thread> pool;
    for (uint32_t t = 0; t < threads; t++) {
        uint32_t n0 = (uint32_t)((uint64_t)N * t / threads);
        uint32_t n1 = (uint32_t)((uint64_t)N * (t + 1) / threads);
        pool.emplace_back([=]() { rows(X, src, bias, Y, M, N, K, n0, n1); });
    }
    for (auto& th : pool) th.join();
}

// ---- any K-quant type the reference's dequant_kquant knows (Q4_K = 12, Q5_K = 13, Q6_K = 14) ----

static uint32_t block_bytes(uint32_t type) { return type == 12 ? 144u : type == 13 ? 176u : type == 14 ? 210u : 0u; }

// dequant_kquant -- runtime/gguf_loader.cpp:455-573
void ref_kq_dequant(uint32_t type, const void* raw, float* out, uint32_t N, uint32_t K) {
    dequant_kquant(raw, out, N, K, (GGUFType)type);
}

// pack_q4k / pack_q5k / pack_q6k -- runtime/gguf_loader.cpp:359-424
void ref_kq_pack(uint32_t type, const void* raw, uint32_t N, uint32_t K, uint32_t* words,
                 uint32_t* rowStrideWords, uint32_t* nBlocks) {
    KQuantPacked p = type == 13 ? pack_q5k(raw, N, K) : type == 14 ? pack_q6k(raw, N, K) : pack_q4k(raw, N, K);
    if (rowStrideWords) *rowStrideWords = p.rowStrideWords;
    if (nBlocks) *nBlocks = p.nBlocks;
    if (words) std::memcpy(words, p.data.data(), p.data.size() * sizeof(uint32_t));
}

// Expected-value computation of the Q5_K / Q6_K kernel tests (runtime/tests/kernel_test.cpp:
// 1669-1676, 1691-1698, 1732-1742): same loops as above, any type.
static void kq_rows(uint32_t type, const float* X, const uint8_t* raw, const float* bias, float* Y,
                    uint32_t M, uint32_t N, uint32_t K, uint32_t n0, uint32_t n1) {
    const uint32_t nb = K / 256, SLAB = 64, bb = block_bytes(type);
    std::vector<float> deq((size_t)SLAB * K);
    for (uint32_t s0 = n0; s0 < n1; s0 += SLAB) {
        const uint32_t cnt = (n1 - s0 < SLAB) ? n1 - s0 : SLAB;
        dequant_kquant(raw + (size_t)s0 * nb * bb, deq.data(), cnt, K, (GGUFType)type);
        for (uint32_t m = 0; m < M; m++)
            for (uint32_t r = 0; r < cnt; r++) {
                const uint32_t n = s0 + r;
                float a = bias ? bias[n] : 0.0f;
                for (uint32_t k = 0; k < K; k++) a += X[(size_t)m * K + k] * deq[(size_t)r * K + k];
                Y[(size_t)m * N + n] = a;
            }
    }
}

void ref_kq_matmul(uint32_t type, const float* X, const void* raw, const float* bias, float* Y,
                   uint32_t M, uint32_t N, uint32_t K, uint32_t threads) {
    const uint8_t* src = (const uint8_t*)raw;
    if (!block_bytes(type)) return;
    if (threads <= 1 || N < threads) {
        kq_rows(type, X, src, bias, Y, M, N, K, 0, N);
        return;
    }
    std::vector<std::thread> pool;
    for (uint32_t t = 0; t < threads; t++) {
        uint32_t n0 = (uint32_t)((uint64_t)N * t / threads);
        uint32_t n1 = (uint32_t)((uint64_t)N * (t + 1) / threads);
        pool.emplace_back([=]() { kq_rows(type, X, src, bias, Y, M, N, K, n0, n1); });
    }
    for (auto& th : pool) th.join();
}

// ---- the reference's GGUF reader (GGUFFile::open and accessors, runtime/gguf_loader.cpp:14-182) ----

void* ref_gguf_open(const char* path) {
    GGUFFile* f = new GGUFFile();
    if (!f->open(path)) {
        delete f;
        return nullptr;
    }
    return f;
}
void ref_gguf_close(void* p) { delete static_cast<GGUFFile*>(p); }
uint32_t ref_gguf_version(void* p) { return static_cast<GGUFFile*>(p)->version; }
uint64_t ref_gguf_n_tensors(void* p) { return static_cast<GGUFFile*>(p)->n_tensors; }
uint64_t ref_gguf_data_offset(void* p) { return static_cast<GGUFFile*>(p)->data_offset; }
int ref_gguf_tensor(void* p, uint64_t i, char* name, uint64_t cap, uint32_t* n_dims, uint64_t* shape4, uint32_t* type,
                    uint64_t* offset) {
    GGUFFile* f = static_cast<GGUFFile*>(p);
    if (i >= f->tensors.size()) return -1;
    const GGUFTensorInfo& t = f->tensors[i];
    std::snprintf(name, cap, "%s", t.name.c_str());
    *n_dims = (uint32_t)t.shape.size();
    for (size_t d = 0; d < 4; d++) shape4[d] = d < t.shape.size() ? t.shape[d] : 1;
    *type = (uint32_t)t.type;
    *offset = t.offset;
    return 0;
}
int ref_gguf_has_key(void* p, const char* key) { return static_cast<GGUFFile*>(p)->hasKey(key) ? 1 : 0; }
uint32_t ref_gguf_get_u32(void* p, const char* key, uint32_t def) { return static_cast<GGUFFile*>(p)->getU32(key, def); }
float ref_gguf_get_f32(void* p, const char* key, float def) { return static_cast<GGUFFile*>(p)->getFloat(key, def); }
int ref_gguf_get_bool(void* p, const char* key, int def) { return static_cast<GGUFFile*>(p)->getBool(key, def != 0) ? 1 : 0; }
int64_t ref_gguf_get_string(void* p, const char* key, int64_t index, char* buf, uint64_t cap) {
    GGUFFile* f = static_cast<GGUFFile*>(p);
    std::string s;
    if (index < 0) {
        if (!f->hasKey(key)) return -1;
        s = f->getString(key, "\x01absent");
        if (s == "\x01absent") return -1;
    } else {
        const std::vector<std::string>* a = f->getStringArray(key);
        if (!a || (uint64_t)index >= a->size()) return -1;
        s = (*a)[index];
    }
    std::snprintf(buf, cap, "%s", s.c_str());
    return (int64_t)s.size();
}
int64_t ref_gguf_i32_array(void* p, const char* key, int32_t* out, uint64_t cap) {
    const std::vector<int32_t>* a = static_cast<GGUFFile*>(p)->getI32Array(key);
    if (!a) return -1;
    for (uint64_t i = 0; i < a->size() && i < cap; i++) out[i] = (*a)[i];
    return (int64_t)a->size();
}

// extractModelConfig (runtime/gguf_loader.cpp:184-317) through a plain struct: the fields of the reference's
// ModelConfig in the order of the library's bpq4k_model_config (tests compare the two byte for byte).
struct ref_model_config {
    char arch[64];
    uint32_t nLayer, nHead, nKvHeads, nEmbd, intermediateSize, nVocab, headDim, kvHeadDim;
    float rmsNormEps, ropeTheta;
    int32_t tieWordEmbeddings, hasQkNorm;
    int32_t activation;
    float embeddingScale, logitSoftcap;
    uint32_t slidingWindow, nLayerAttnTypes;
    int32_t hasSandwichNorm;
    uint32_t pleSize, sharedKvLayers;
    int32_t hasMtp;
    uint32_t mtpNumLayers;
    uint32_t numExperts, numExpertsPerTok, moeIntermediateSize, moeSharedIntermediateSize;
    uint32_t ssmInnerSize, ssmStateSize, ssmConvKernel, ssmGroupCount, ssmTimeStepRank, fullAttentionInterval;
    int32_t ropeSections[4];
};
int ref_extract_model_config(void* p, ref_model_config* c, uint8_t* layer_attn_types, uint32_t cap) {
    const ModelConfig m = extractModelConfig(*static_cast<GGUFFile*>(p));
    std::memset(c, 0, sizeof(*c));
    std::snprintf(c->arch, sizeof(c->arch), "%s", m.arch.c_str());
    c->nLayer = m.nLayer; c->nHead = m.nHead; c->nKvHeads = m.nKvHeads; c->nEmbd = m.nEmbd;
    c->intermediateSize = m.intermediateSize; c->nVocab = m.nVocab; c->headDim = m.headDim; c->kvHeadDim = m.kvHeadDim;
    c->rmsNormEps = m.rmsNormEps; c->ropeTheta = m.ropeTheta;
    c->tieWordEmbeddings = m.tieWordEmbeddings; c->hasQkNorm = m.hasQkNorm;
    c->activation = m.activation == ActivationType::GELU ? 1 : 0;
    c->embeddingScale = m.embeddingScale; c->logitSoftcap = m.logitSoftcap;
    c->slidingWindow = m.slidingWindow; c->nLayerAttnTypes = (uint32_t)m.layerAttnTypes.size();
    for (uint32_t i = 0; i < m.layerAttnTypes.size() && layer_attn_types && i < cap; i++)
        layer_attn_types[i] = m.layerAttnTypes[i] == AttnLayerType::SlidingWindow ? 1 : 0;
    c->hasSandwichNorm = m.hasSandwichNorm; c->pleSize = m.pleSize; c->sharedKvLayers = m.sharedKvLayers;
    c->hasMtp = m.hasMtp; c->mtpNumLayers = m.mtpNumLayers;
    c->numExperts = m.numExperts; c->numExpertsPerTok = m.numExpertsPerTok;
    c->moeIntermediateSize = m.moeIntermediateSize; c->moeSharedIntermediateSize = m.moeSharedIntermediateSize;
    c->ssmInnerSize = m.ssmInnerSize; c->ssmStateSize = m.ssmStateSize; c->ssmConvKernel = m.ssmConvKernel;
    c->ssmGroupCount = m.ssmGroupCount; c->ssmTimeStepRank = m.ssmTimeStepRank; c->fullAttentionInterval = m.fullAttentionInterval;
    for (int i = 0; i < 4; i++) c->ropeSections[i] = i < (int)m.ropeSections.size() ? m.ropeSections[i] : 0;
    return 0;
}

}  // extern "C"
