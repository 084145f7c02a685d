// Reference arm of the benchmark, decode steps at a standing context: the reference's own
// LLMEngine (engine/include/llm_engine.h:27-56) with its Qwen3ModelRunner on the GPU, configured
// as its command line configures it (model/model_main.cpp:276-303: token budget min(max_seq_len,
// 256), pages of 16), driven through add_request() and step().  Nothing of the engine under test
// is linked in.  The prompts are prefilled outside the timed region; then WARMUP untimed and STEPS
// timed steps in which every request decodes one token (step() returns only when the sampled
// tokens are on the host, so the wall clock around it is the step's time).
//
// usage: decode_main MODEL.safetensors TOKENIZER.json BATCH PROMPT_LEN WARMUP STEPS MAX_SEQ_LEN NUM_KV_BLOCKS MAX_TOKEN_ID SEED
// prints one line: {"batch":..,"prompt_len":..,"steps":..,"seconds":..,"tokens_per_second":..,"ms_per_step":..,"prefill_seconds":..}
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <vector>

#include "llm_engine.h"
#include "qwen3.h"
#include "qwen3_runner.h"

using namespace my_vllm;
using namespace my_vllm::engine;

static int fail(const char* what, const Status& s) {
    fprintf(stderr, "decode_main: %s: %s\n", what, s.get_err_msg().c_str());
    return 1;
}

int main(int argc, char** argv) {
    if (argc != 11) {
        fprintf(stderr, "usage: decode_main MODEL TOKENIZER BATCH PROMPT_LEN WARMUP STEPS MAX_SEQ_LEN NUM_KV_BLOCKS MAX_TOKEN_ID SEED\n");
        return 2;
    }
    const std::string model_path = argv[1], tokenizer = argv[2];
    const int batch = atoi(argv[3]), prompt_len = atoi(argv[4]), warmup = atoi(argv[5]), steps = atoi(argv[6]);
    const int max_seq_len = atoi(argv[7]), num_blocks = atoi(argv[8]), max_token_id = atoi(argv[9]);
    const uint64_t seed = strtoull(argv[10], nullptr, 10);

    Qwen3Model model(tokenizer, model_path, max_seq_len);
    Status s = model.set_weight_quantization(0);
    if (!s) return fail("quantization", s);
    fprintf(stderr, "decode_main: loading the model...\n");
    s = model.init(DeviceType::kDeviceCUDA);
    if (!s) return fail("model.init", s);

    Qwen3ModelRunner runner(model);
    EngineConfig config;
    config.max_model_len = max_seq_len;
    config.scheduler.max_num_seqs = batch;
    config.scheduler.max_num_batched_tokens = std::min<int32_t>(max_seq_len, 256);
    config.scheduler.block_size = std::min<int32_t>(16, max_seq_len);
    config.scheduler.num_kv_blocks = num_blocks;
    LLMEngine engine(runner, config);
    s = engine.init();
    if (!s) return fail("engine.init", s);

    // the prompts of the reference's own benchmark: uniform ids from a seeded mt19937_64, temperature
    // 0.6, end-of-sequence ignored, per-request seed (model/model_main.cpp:150-175)
    std::mt19937_64 rng(seed);
    std::uniform_int_distribution<int32_t> token_id(0, std::min(max_token_id, model.vocab_size() - 1));
    const int budget_steps = (batch * prompt_len + config.scheduler.max_num_batched_tokens - 1) /
                             config.scheduler.max_num_batched_tokens;
    for (int i = 0; i < batch; ++i) {
        std::vector<int32_t> prompt(static_cast<size_t>(prompt_len));
        std::generate(prompt.begin(), prompt.end(), [&] { return token_id(rng); });
        SamplingParams sampling;
        sampling.temperature = 0.6f;
        sampling.ignore_eos = true;
        sampling.max_tokens = warmup + steps + budget_steps + budget_steps / 8 + 16;   // nobody finishes inside the timed region
        sampling.seed = seed + static_cast<uint64_t>(i) + 1;
        uint64_t id = 0;
        s = engine.add_request(prompt, sampling, id);
        if (!s) return fail("add_request", s);
    }

    std::vector<GenerationResult> done;
    const auto t_prefill = std::chrono::steady_clock::now();
    int prefill_steps = 0;
    while (true) {            // until a step is decode only: every request makes one token in it
        const uint64_t before = engine.total_generated_tokens();
        s = engine.step(done);
        if (!s) return fail("step (prefill)", s);
        ++prefill_steps;
        if (!done.empty()) { fprintf(stderr, "decode_main: a request finished during the prompts\n"); return 1; }
        if (engine.total_generated_tokens() - before == static_cast<uint64_t>(batch) && prefill_steps >= budget_steps) break;
        if (prefill_steps % 10 == 0) fprintf(stderr, "decode_main: %d prompt steps...\n", prefill_steps);
        if (prefill_steps > 4 * budget_steps + 16) { fprintf(stderr, "decode_main: the prompts do not end\n"); return 1; }
    }
    const double prefill_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_prefill).count();
    for (int i = 0; i < warmup; ++i) {
        s = engine.step(done);
        if (!s) return fail("step (warm-up)", s);
    }
    const uint64_t generated_before = engine.total_generated_tokens();
    const auto started = std::chrono::steady_clock::now();
    for (int i = 0; i < steps; ++i) {
        s = engine.step(done);
        if (!s) return fail("step", s);
        if (!done.empty()) { fprintf(stderr, "decode_main: a request finished inside the timed region\n"); return 1; }
    }
    const double seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - started).count();
    const uint64_t generated = engine.total_generated_tokens() - generated_before;
    if (generated != static_cast<uint64_t>(batch) * steps) {
        fprintf(stderr, "decode_main: %llu tokens in %d steps of %d requests\n", (unsigned long long)generated, steps, batch);
        return 1;
    }
    printf("{\"batch\": %d, \"prompt_len\": %d, \"steps\": %d, \"warmup\": %d, \"seconds\": %.6f, \"tokens_per_second\": %.3f, "
           "\"ms_per_step\": %.4f, \"prefill_seconds\": %.3f, \"prefill_steps\": %d}\n",
           batch, prompt_len, steps, warmup, seconds, generated / seconds, 1e3 * seconds / steps, prefill_seconds, prefill_steps);
    fflush(stdout);
    return 0;
}
