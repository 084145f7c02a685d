// Golden run, part 1: the reference's own Qwen3Model on the CPU, one whole prompt through
// forward_paged_batch with a scrambled page table, logits of every row to a file.
// usage: logits_main MODEL_DIR OUT.bin PAGE_SIZE NUM_PAGES MAX_SEQ_LEN id0 id1 ...
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "qwen3.h"
int main(int argc, char** argv) {
    std::string dir = argv[1];
    const int page = atoi(argv[3]), pages = atoi(argv[4]), max_seq_len = atoi(argv[5]);
    std::vector<int32_t> toks;
    for (int i = 6; i < argc; ++i) toks.push_back(atoi(argv[i]));
    my_vllm::Qwen3Model model(dir + "/tokenizer.json", dir + "/model.safetensors", max_seq_len);
    my_vllm::Status s = model.init(my_vllm::DeviceType::kDeviceCPU);
    if (!s) { fprintf(stderr, "init: %s\n", s.get_err_msg().c_str()); return 1; }
    s = model.configure_paged_kv_cache(pages, page, max_seq_len);
    if (!s) { fprintf(stderr, "kv: %s\n", s.get_err_msg().c_str()); return 1; }
    std::vector<int32_t> table;                       // pages handed out from the top, odd ones first
    for (int p = pages - 1; p >= 0; --p) if (p % 2) table.push_back(p);
    for (int p = pages - 1; p >= 0; --p) if (p % 2 == 0) table.push_back(p);
    std::vector<int32_t> pos; std::vector<std::vector<int32_t>> tables; std::vector<size_t> rows;
    for (size_t i = 0; i < toks.size(); ++i) { pos.push_back((int)i); tables.push_back(table); rows.push_back(i); }
    std::vector<std::vector<float>> logits;
    s = model.forward_paged_batch(toks, pos, tables, rows, logits);
    if (!s) { fprintf(stderr, "forward: %s\n", s.get_err_msg().c_str()); return 1; }
    FILE* f = fopen(argv[2], "wb");
    for (auto& r : logits) fwrite(r.data(), sizeof(float), r.size(), f);
    fclose(f);
    printf("rows=%zu vocab=%zu\n", logits.size(), logits[0].size());
    return 0;
}
