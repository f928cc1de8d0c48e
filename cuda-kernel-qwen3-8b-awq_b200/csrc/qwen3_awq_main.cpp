// Example harness: the reference's main (Inference.cu:1413-1433) on the rebuilt class.
//   qwen3_awq_infer <weight_dir> [max_new_tokens] [n_gpus] [layers hidden inter vocab max_pos]
// Prompt is the single BOS id 151643 (Inference.cu:1422) when it fits the vocabulary, else 0.
#include <cstdio>
#include <cstdlib>
#include <iostream>

#include "../../include/qwen3_awq_infer.h"

int main(int argc, char** argv) {
    if (argc < 2) {
        std::cerr << "Usage: " << argv[0] << " <path_to_weight_folder> [max_new_tokens] [n_gpus] [layers hidden inter vocab max_pos]\n";
        return 1;
    }
    Qw3Config cfg;
    qw3_config_default(&cfg);
    const int max_new_tokens = argc > 2 ? std::atoi(argv[2]) : 20;
    if (argc > 3) {
        cfg.n_stages = std::atoi(argv[3]);
        for (int s = 0; s < cfg.n_stages && s < QW3_MAX_STAGES; ++s) cfg.device[s] = s;
    }
    if (argc > 8) {
        cfg.layers = std::atoi(argv[4]); cfg.hidden = std::atoi(argv[5]); cfg.inter = std::atoi(argv[6]);
        cfg.vocab = std::atoi(argv[7]); cfg.max_pos = std::atoi(argv[8]);
        cfg.heads = cfg.hidden / 128;
    }
    try {
        QWen3AWQInfer infer(argv[1], cfg);
        std::vector<int> prompt = {151643 < cfg.vocab ? 151643 : 0};
        std::vector<int> out = infer.generateResponse(prompt, max_new_tokens);
        std::cout << "Generated tokens: ";
        for (int tok : out) std::cout << tok << " ";
        std::cout << std::endl;
    } catch (const std::exception& e) {
        std::cerr << "ERROR: " << e.what() << "\n";
        return 1;
    }
    return 0;
}
