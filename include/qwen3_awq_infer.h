/*
 * QWen3AWQInfer: the reference's public class (Inference.cu:356-366) rebuilt on the C ABI of
 * qw3_cabi.h.  Header-only; link against libqw3awq.so.
 *
 *   QWen3AWQInfer infer(weight_dir);                         // Inference.cu:358, 1419
 *   std::vector<int> ids = infer.generateResponse(prompt, 20); // Inference.cu:364, 1425
 *
 * Differences a caller can observe: failures throw std::runtime_error instead of printing and
 * calling std::exit(1) (Inference.cu:52-71, 299-308, 566-578); the object can be reused for
 * several prompts (the reference never resets current_seq_len_, Inference.cu:430); a second
 * constructor takes a Qw3Config (stage split over 1..8 GPUs, rope base, KV capacity, ...).
 * The object owns every device allocation and is movable but not copyable.
 */
#ifndef QWEN3_AWQ_INFER_H
#define QWEN3_AWQ_INFER_H

#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "qw3_cabi.h"

class QWen3AWQInfer {
public:
    explicit QWen3AWQInfer(const std::string& weight_dir) {
        Qw3Config cfg;
        qw3_config_default(&cfg);
        open(weight_dir, cfg);
    }
    QWen3AWQInfer(const std::string& weight_dir, const Qw3Config& cfg) { open(weight_dir, cfg); }
    ~QWen3AWQInfer() { qw3_destroy(h_); }

    QWen3AWQInfer(const QWen3AWQInfer&) = delete;
    QWen3AWQInfer& operator=(const QWen3AWQInfer&) = delete;
    QWen3AWQInfer(QWen3AWQInfer&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
    QWen3AWQInfer& operator=(QWen3AWQInfer&& o) noexcept {
        if (this != &o) {
            qw3_destroy(h_);
            h_ = o.h_;
            o.h_ = nullptr;
        }
        return *this;
    }

    // prompt_ids: input token IDs; max_new_tokens: how many to generate; returns only the newly
    // generated token IDs (Inference.cu:361-366).
    std::vector<int> generateResponse(const std::vector<int>& prompt_ids, int max_new_tokens) {
        std::vector<int32_t> prompt(prompt_ids.begin(), prompt_ids.end());
        std::vector<int32_t> out(max_new_tokens > 0 ? max_new_tokens : 0);
        int32_t n_out = 0;
        check(qw3_generate(h_, prompt.data(), (int32_t)prompt.size(), max_new_tokens, out.data(), &n_out), "generateResponse");
        return std::vector<int>(out.begin(), out.begin() + n_out);
    }

    // Device time of the last call's prompt loop and decode loop, in milliseconds.
    std::pair<float, float> lastTiming() const {
        float a = 0.f, b = 0.f;
        qw3_last_timing(h_, &a, &b);
        return {a, b};
    }

    qw3_handle handle() const { return h_; }

private:
    void open(const std::string& dir, const Qw3Config& cfg) { check(qw3_create(dir.c_str(), &cfg, &h_), "QWen3AWQInfer"); }
    static void check(int status, const char* where) {
        if (status != QW3_OK)
            throw std::runtime_error(std::string(where) + ": " + qw3_strerror(status) + " (" + qw3_last_error() + ")");
    }
    qw3_handle h_ = nullptr;
};

#endif
