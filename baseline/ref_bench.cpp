// The reference arm of bench.py: tattooinmtl/Ultima.cpp's own model code (compiled unchanged, for
// the CPU it is written for) through its public interface: load_model on a LoadedModel, a KVCache,
// IModel::prefill and IModel::decode, its sampler's argmax.  The model is Qwen3 dense at the layer
// sizes given on the command line, weights random from a counter hash, stored as BF16 (norm
// weights F32), held in memory: the reference's file loader is for Windows only, so the model
// reaches it through its abstract LoadedModel, as its own configuration tests do
// (tests/unit/test_qwen_config.cpp:18-38).  It has no batch: the sequences of a batch run one after
// another, which is how a user of the reference would serve them (apps/ultima-cli/main.cpp:652-686).
// Timing is the reference's own way: steady_clock around the prefill and around the decode loop
// (apps/ultima-cli/main.cpp:654-698).
//
//   ref_bench LAYERS HIDDEN FFN HEADS KV_HEADS HEAD_DIM VOCAB BATCH PROMPT STEPS WARMUP PREFILL_TOKENS THREADS
//
// Prints one line: decode_tokens_per_s prefill_tokens_per_s ms_per_step prefill_ms
#include "ultima/kv_cache/kv_cache.hpp"
#include "ultima/model/imodel.hpp"
#include "ultima/model/loaded_model.hpp"
#include "ultima/runtime/thread_pool.hpp"
#include "ultima/sampler/sampler.hpp"

#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <span>
#include <string>
#include <vector>

using namespace ultima::model;

static std::uint64_t mix64(std::uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// about normal: the sum of four uniform numbers, scaled to unit variance
static float near_normal(std::uint64_t key, std::uint64_t i) {
    const std::uint64_t r = mix64(key ^ mix64(i));
    const float s = (float)(r & 0xFFFF) + (float)((r >> 16) & 0xFFFF) + (float)((r >> 32) & 0xFFFF) + (float)(r >> 48);
    return (s / 65536.0f - 2.0f) * 1.7320508f;
}
static std::uint16_t to_bf16(float v) {
    std::uint32_t u;
    std::memcpy(&u, &v, 4);
    return (std::uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

struct Mem : LoadedModel {
    std::string arch = "qwen3";
    MetadataStore md;
    std::vector<TensorInfo> infos;
    std::map<std::string, std::vector<std::uint8_t>, std::less<>> data;

    void add(const std::string& name, std::vector<std::uint64_t> dims_inner_first, bool vector_f32, float shift, float stdv) {
        std::uint64_t n = 1;
        for (auto d : dims_inner_first) n *= d;
        TensorInfo ti;
        ti.name = name; ti.dims = dims_inner_first; ti.offset = 0;
        ti.dtype = vector_f32 ? DataType::F32 : DataType::BF16;
        ti.size_bytes = n * (vector_f32 ? 4 : 2);
        std::vector<std::uint8_t> bytes(ti.size_bytes);
        const std::uint64_t key = mix64(std::hash<std::string>{}(name));
        if (vector_f32) {
            float* p = reinterpret_cast<float*>(bytes.data());
            for (std::uint64_t i = 0; i < n; ++i) p[i] = shift + stdv * near_normal(key, i);
        } else {
            std::uint16_t* p = reinterpret_cast<std::uint16_t*>(bytes.data());
            for (std::uint64_t i = 0; i < n; ++i) p[i] = to_bf16(shift + stdv * near_normal(key, i));
        }
        infos.push_back(ti);
        data[name] = std::move(bytes);
    }
    const std::string& architecture() const override { return arch; }
    const MetadataStore& metadata() const override { return md; }
    const std::vector<TensorInfo>& tensor_infos() const override { return infos; }
    std::optional<TensorView> tensor(std::string_view name) const override {
        for (const auto& ti : infos)
            if (ti.name == name) return TensorView{ti, data.find(name)->second.data()};
        return std::nullopt;
    }
    std::uint64_t file_size_bytes() const override { return 0; }
    std::uint64_t alignment() const override { return 32; }
    std::uint32_t gguf_version() const override { return 3; }
    const std::uint8_t* file_data() const override { return nullptr; }
};

int main(int argc, char** argv) {
    if (argc != 14) { std::fprintf(stderr, "usage: ref_bench LAYERS HIDDEN FFN HEADS KV_HEADS HEAD_DIM VOCAB BATCH PROMPT STEPS WARMUP PREFILL_TOKENS THREADS\n"); return 2; }
    const std::uint64_t L = std::atoll(argv[1]), H = std::atoll(argv[2]), F = std::atoll(argv[3]), nh = std::atoll(argv[4]),
                        nkv = std::atoll(argv[5]), hd = std::atoll(argv[6]), V = std::atoll(argv[7]);
    const int batch = std::atoi(argv[8]), prompt = std::atoi(argv[9]), steps = std::atoi(argv[10]), warmup = std::atoi(argv[11]),
              prefill_tokens = std::atoi(argv[12]), threads = std::atoi(argv[13]);
    const std::uint64_t ctx = (std::uint64_t)std::max(prompt + steps + warmup + 8, prefill_tokens + 8);

    Mem m;
    m.md.insert("general.architecture", MetadataValue{std::string("qwen3")});
    m.md.insert("qwen3.context_length", MetadataValue{std::uint64_t{ctx}});
    m.md.insert("qwen3.embedding_length", MetadataValue{std::uint64_t{H}});
    m.md.insert("qwen3.block_count", MetadataValue{std::uint64_t{L}});
    m.md.insert("qwen3.feed_forward_length", MetadataValue{std::uint64_t{F}});
    m.md.insert("qwen3.attention.head_count", MetadataValue{std::uint64_t{nh}});
    m.md.insert("qwen3.attention.head_count_kv", MetadataValue{std::uint64_t{nkv}});
    m.md.insert("qwen3.attention.key_length", MetadataValue{std::uint64_t{hd}});
    m.md.insert("qwen3.attention.layer_norm_rms_epsilon", MetadataValue{1e-6f});
    m.md.insert("qwen3.rope.freq_base", MetadataValue{1000000.0f});
    m.md.insert("tokenizer.ggml.tokens", MetadataValue{std::vector<std::string>(V, "x")});
    m.add("token_embd.weight", {H, V}, false, 0.f, 0.02f);
    for (std::uint64_t i = 0; i < L; ++i) {
        const std::string p = "blk." + std::to_string(i) + ".";
        m.add(p + "attn_norm.weight", {H}, true, 1.f, 0.05f);
        m.add(p + "attn_q.weight", {H, nh * hd}, false, 0.f, 0.02f);
        m.add(p + "attn_k.weight", {H, nkv * hd}, false, 0.f, 0.02f);
        m.add(p + "attn_v.weight", {H, nkv * hd}, false, 0.f, 0.02f);
        m.add(p + "attn_q_norm.weight", {hd}, true, 1.f, 0.05f);
        m.add(p + "attn_k_norm.weight", {hd}, true, 1.f, 0.05f);
        m.add(p + "attn_output.weight", {nh * hd, H}, false, 0.f, 0.02f);
        m.add(p + "ffn_norm.weight", {H}, true, 1.f, 0.05f);
        m.add(p + "ffn_gate.weight", {H, F}, false, 0.f, 0.02f);
        m.add(p + "ffn_up.weight", {H, F}, false, 0.f, 0.02f);
        m.add(p + "ffn_down.weight", {F, H}, false, 0.f, 0.02f);
    }
    m.add("output_norm.weight", {H}, true, 1.f, 0.05f);
    m.add("output.weight", {H, V}, false, 0.f, 0.02f);
    std::fprintf(stderr, "[ref_bench] model in memory\n");

    ultima::runtime::ThreadPool pool{(std::size_t)threads};
    auto mr = load_model(m, pool);
    if (!mr) { std::fprintf(stderr, "load_model failed: %s\n", mr.error().message.c_str()); return 4; }
    auto& model = **mr;
    const auto& d = model.dims();
    ultima::kv_cache::KVCache::Config kc;
    kc.n_slots = (std::size_t)batch + 1; kc.n_ctx = ctx; kc.n_layers = d.n_layers; kc.n_kv_heads = d.n_kv_heads;
    kc.head_dim = d.head_dim; kc.dtype = DataType::F32;
    ultima::kv_cache::KVCache kv{kc};
    std::vector<float> logits(V);
    using clock = std::chrono::steady_clock;

    // prefill of one prompt of PREFILL_TOKENS tokens
    std::vector<std::int32_t> long_prompt(prefill_tokens);
    for (int i = 0; i < prefill_tokens; ++i) long_prompt[i] = (std::int32_t)(mix64(77 + i) % V);
    auto s0 = kv.acquire(1000);
    const auto p0 = clock::now();
    if (!model.prefill(kv, s0, std::span<const std::int32_t>(long_prompt), logits.data())) { std::fprintf(stderr, "prefill failed\n"); return 5; }
    const double prefill_ms = std::chrono::duration<double, std::milli>(clock::now() - p0).count();
    kv.release(s0);
    std::fprintf(stderr, "[ref_bench] prefill of %d tokens: %.1f ms\n", prefill_tokens, prefill_ms);

    // a batch of sequences, one after another: their prompts, then one token each a step
    std::vector<ultima::kv_cache::SlotHandle> slots;
    std::vector<std::int32_t> next(batch);
    for (int b = 0; b < batch; ++b) {
        std::vector<std::int32_t> p(prompt);
        for (int i = 0; i < prompt; ++i) p[i] = (std::int32_t)(mix64(1000 * (b + 1) + i) % V);
        slots.push_back(kv.acquire((std::uint64_t)b + 1));
        if (!model.prefill(kv, slots[b], std::span<const std::int32_t>(p), logits.data())) { std::fprintf(stderr, "prefill failed\n"); return 5; }
        next[b] = (std::int32_t)ultima::sampler::argmax(logits);
    }
    auto one_step = [&]() {
        for (int b = 0; b < batch; ++b) {
            if (!model.decode(kv, slots[b], next[b], logits.data())) { std::fprintf(stderr, "decode failed\n"); std::exit(5); }
            next[b] = (std::int32_t)ultima::sampler::argmax(logits);
        }
    };
    for (int i = 0; i < warmup; ++i) one_step();
    const auto t0 = clock::now();
    for (int i = 0; i < steps; ++i) one_step();
    const double ms = std::chrono::duration<double, std::milli>(clock::now() - t0).count();
    std::printf("%.4f %.4f %.4f %.4f\n", batch * steps / ms * 1e3, prefill_tokens / prefill_ms * 1e3, ms / steps, prefill_ms);
    return 0;
}
