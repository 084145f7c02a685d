// Golden run, part 2: the reference's LLMEngine on the CPU with token-id requests: greedy
// tokens and the number of steps under a token budget and a number of pages.
// usage: engine_main MODEL_DIR BUDGET NUM_PAGES MAX_TOKENS PAGE_SIZE MAX_MODEL_LEN id,id,... [more prompts]
#include <cstdio>
#include <cstdlib>
#include <sstream>
#include "llm_engine.h"
#include "qwen3.h"
#include "qwen3_runner.h"
using namespace my_vllm; using namespace my_vllm::engine;
int main(int argc, char** argv) {
    std::string dir = argv[1]; int budget = atoi(argv[2]), blocks = atoi(argv[3]), max_tokens = atoi(argv[4]);
    const int page = atoi(argv[5]), max_len = atoi(argv[6]);
    Qwen3Model model(dir + "/tokenizer.json", dir + "/model.safetensors", max_len);
    Status s = model.init(DeviceType::kDeviceCPU); if (!s) { puts(s.get_err_msg().c_str()); return 1; }
    Qwen3ModelRunner runner(model); EngineConfig cfg; cfg.max_model_len = max_len;
    cfg.scheduler.max_num_seqs = 4; cfg.scheduler.max_num_batched_tokens = budget;
    cfg.scheduler.block_size = page; cfg.scheduler.num_kv_blocks = blocks;
    LLMEngine engine(runner, cfg); s = engine.init(); if (!s) { puts(s.get_err_msg().c_str()); return 1; }
    for (int a = 7; a < argc; ++a) {
        std::vector<int32_t> p; std::stringstream ss(argv[a]); std::string item;
        while (std::getline(ss, item, ',')) p.push_back(atoi(item.c_str()));
        SamplingParams sp; sp.max_tokens = max_tokens; sp.ignore_eos = true; uint64_t id;
        s = engine.add_request(p, sp, id); if (!s) { puts(s.get_err_msg().c_str()); return 1; }
    }
    std::vector<GenerationResult> done; int steps = 0;
    while (!engine.is_finished()) {
        s = engine.step(done); if (!s) { printf("error %s\n", s.get_err_msg().c_str()); return 1; } ++steps;
        for (auto& r : done) { printf("req %lu", (unsigned long)r.request_id); for (int t : r.token_ids) printf(" %d", t); printf("\n"); }
    }
    printf("steps %d\n", steps);
    return 0;
}
