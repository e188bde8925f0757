// bmb_train_gpt -- a training driver over the C ABI of libbmb.so that speaks the reference
// trainer's dialect: the flags of src/train_gpt.cu:229-277, its report lines before training
// (data / model / params / memory / total, src/train_gpt.cu:322-355, which tools/flash_memory.py
// parses under --alloc-only), its step line (src/train_gpt.cu:476-485, which tools/plot_training.py
// parses), its [eval] lines, GPT1 checkpoints (--save / --load) and sampling.
//
// What the reference's command line cannot say is added as flags: --heads, --embd, --beta1,
// --beta2, --wd, --synthetic with --vocab (token ids uniform over a vocabulary instead of a text
// file), --math fp32|tf32|bf16, --fused 0|1, and --resume (a checkpoint with optimiser state:
// parameters, AdamW moments and the step counter continue where they stopped).
//
// Host code only: plain C++ linked against libbmb.so; every device operation happens behind the
// bmb_trainer_* entry points (one stream, forward + backward replayed from a CUDA graph, the loss
// read asynchronously).  One GPU per process; data-parallel runs use one process per GPU with a
// communicator attached to each trainer, which bench.py's launcher shows.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "bmb.h"

namespace {

struct Options {
    const char *data_path = "data/input.txt";
    int steps = 2000, B = 16, T = 256, n_layer = 6, n_head = 6, n_embd = 384;
    float lr = 1e-3f, weight_decay = 0.1f, grad_clip = 1.0f, beta1 = 0.9f, beta2 = 0.999f;
    int warmup = 100, eval_every = 100, sample_every = 500, sample_len = 400, eval_batches = 20;
    const char *save_path = "bench/gpt.bin";
    const char *load_path = nullptr, *resume_path = nullptr;
    float temperature = 0.8f;
    unsigned seed = 1337;
    bool use_flash = true, alloc_only = false, synthetic = false, save_optimizer = false;
    int synthetic_vocab = 50304, math = BMB_MATH_FP32, fused = -1;
};

[[noreturn]] void die(const char *what) {
    fprintf(stderr, "%s: %s\n", what, bmb_last_error());
    exit(1);
}
#define CHECK(call) do { if ((call) != BMB_OK) die(#call); } while (0)

struct Corpus {
    std::vector<int> train, val;
    std::string itos;            // token id -> byte
};

// Character-level corpus: the vocabulary is the sorted set of bytes present, the last tenth of the
// text is held out (src/train_gpt.cu:110-143).
Corpus read_text(const char *path, float val_frac) {
    FILE *f = fopen(path, "rb");
    if (!f) { fprintf(stderr, "cannot open %s\n", path); exit(1); }
    std::string text;
    char buf[1 << 16];
    size_t got;
    while ((got = fread(buf, 1, sizeof buf, f)) > 0) text.append(buf, got);
    fclose(f);
    int id_of[256];
    bool seen[256] = {false};
    for (unsigned char ch : text) seen[ch] = true;
    Corpus c;
    for (int b = 0; b < 256; ++b) {
        id_of[b] = -1;
        if (seen[b]) { id_of[b] = (int)c.itos.size(); c.itos.push_back((char)b); }
    }
    const size_t nval = (size_t)(text.size() * val_frac), ntrain = text.size() - nval;
    c.train.reserve(ntrain);
    c.val.reserve(nval);
    for (size_t i = 0; i < text.size(); ++i) (i < ntrain ? c.train : c.val).push_back(id_of[(unsigned char)text[i]]);
    return c;
}

// B windows of T+1 tokens at random offsets: inputs [0,T), targets [1,T+1) (src/train_gpt.cu:146-157).
void draw_windows(const std::vector<int> &data, int B, int T, std::mt19937 &rng, std::vector<int> &x, std::vector<int> &y) {
    std::uniform_int_distribution<size_t> pick(0, data.size() - T - 2);
    for (int b = 0; b < B; ++b) {
        const size_t off = pick(rng);
        for (int t = 0; t < T; ++t) {
            x[(size_t)b * T + t] = data[off + t];
            y[(size_t)b * T + t] = data[off + t + 1];
        }
    }
}

// Token ids and targets uniform over the vocabulary (tools/test_grad.cu:72-75 draws its batch this way).
void draw_uniform(int vocab, std::mt19937 &rng, std::vector<int> &x, std::vector<int> &y) {
    std::uniform_int_distribution<int> d(0, vocab - 1);
    for (auto &v : x) v = d(rng);
    for (auto &v : y) v = d(rng);
}

// Linear warm-up, then cosine decay to a tenth of the peak (src/train_gpt.cu:233-238).
float lr_at(int step, int warmup, int total, float peak) {
    const float floor_lr = 0.1f * peak;
    if (step <= warmup) return peak * (float)step / (float)warmup;
    const float p = (float)(step - warmup) / (float)std::max(1, total - warmup);
    return floor_lr + 0.5f * (peak - floor_lr) * (1.0f + cosf(3.14159265f * p));
}

struct Run {
    Options o;
    Corpus corpus;
    bmb_trainer *t = nullptr;
    int V = 0, Vp = 0;

    void batch(bool validation, std::mt19937 &rng, std::vector<int> &x, std::vector<int> &y) {
        if (o.synthetic) draw_uniform(V, rng, x, y);
        else draw_windows(validation ? corpus.val : corpus.train, o.B, o.T, rng, x, y);
    }
    // Mean loss over n_batches windows drawn from a generator of its own (src/train_gpt.cu:163-173).
    float evaluate(bool validation, unsigned seed, int n_batches) {
        std::mt19937 erng(seed);
        std::vector<int> x((size_t)o.B * o.T), y((size_t)o.B * o.T);
        double total = 0.0;
        for (int i = 0; i < n_batches; ++i) {
            batch(validation, erng, x, y);
            CHECK(bmb_trainer_upload(t, x.data(), y.data()));
            float loss = 0.0f;
            CHECK(bmb_trainer_forward_loss(t, &loss));
            total += loss;
        }
        return (float)(total / n_batches);
    }
    std::string sample(int len, unsigned seed) {
        int start = 0;
        for (size_t i = 0; i < corpus.itos.size(); ++i)
            if (corpus.itos[i] == '\n') { start = (int)i; break; }
        std::vector<int> toks((size_t)std::max(len, 1));
        CHECK(bmb_trainer_generate(t, start, len, seed, o.temperature, toks.data()));
        std::string s;
        for (int i = 0; i < len; ++i) s.push_back((size_t)toks[i] < corpus.itos.size() ? corpus.itos[toks[i]] : '?');
        return s;
    }
};

bmb_train_config make_config(const Options &o, int T, int V, int Vp, int L, int NH, int C) {
    bmb_train_config c{};
    c.max_seq_len = T; c.vocab_size = V; c.padded_vocab = Vp; c.n_layer = L; c.n_head = NH; c.n_embd = C;
    c.B = o.B; c.T = T; c.use_flash = o.use_flash ? 1 : 0; c.math = o.math;
    c.fused = o.fused >= 0 ? o.fused : (o.math == BMB_MATH_TF32 ? 1 : 0);
    c.beta1 = o.beta1; c.beta2 = o.beta2; c.eps = 1e-8f; c.weight_decay = o.weight_decay; c.grad_clip = o.grad_clip;
    return c;
}

}  // namespace

int main(int argc, char **argv) {
    Run run;
    Options &o = run.o;
    for (int i = 1; i < argc; ++i) {
        const char *a = argv[i];
        auto val = [&]() -> const char * {
            if (i + 1 >= argc) { fprintf(stderr, "%s needs a value\n", a); exit(1); }
            return argv[++i];
        };
        if (!strcmp(a, "-d")) o.data_path = val();
        else if (!strcmp(a, "-n")) o.steps = atoi(val());
        else if (!strcmp(a, "-b")) o.B = atoi(val());
        else if (!strcmp(a, "-t")) o.T = atoi(val());
        else if (!strcmp(a, "-l")) o.n_layer = atoi(val());
        else if (!strcmp(a, "--heads")) o.n_head = atoi(val());
        else if (!strcmp(a, "--embd")) o.n_embd = atoi(val());
        else if (!strcmp(a, "--lr")) o.lr = (float)atof(val());
        else if (!strcmp(a, "--warmup")) o.warmup = atoi(val());
        else if (!strcmp(a, "--clip")) o.grad_clip = (float)atof(val());
        else if (!strcmp(a, "--wd")) o.weight_decay = (float)atof(val());
        else if (!strcmp(a, "--beta1")) o.beta1 = (float)atof(val());
        else if (!strcmp(a, "--beta2")) o.beta2 = (float)atof(val());
        else if (!strcmp(a, "--eval")) o.eval_every = atoi(val());
        else if (!strcmp(a, "--sample")) o.sample_every = atoi(val());
        else if (!strcmp(a, "--seed")) o.seed = (unsigned)atoi(val());
        else if (!strcmp(a, "--eval-batches")) o.eval_batches = atoi(val());
        else if (!strcmp(a, "--save")) o.save_path = val();
        else if (!strcmp(a, "--save-optimizer")) o.save_optimizer = true;
        else if (!strcmp(a, "--load")) o.load_path = val();
        else if (!strcmp(a, "--resume")) o.resume_path = val();
        else if (!strcmp(a, "--len")) o.sample_len = atoi(val());
        else if (!strcmp(a, "--temp")) o.temperature = (float)atof(val());
        else if (!strcmp(a, "--alloc-only")) o.alloc_only = true;
        else if (!strcmp(a, "--unfused")) o.use_flash = false;
        else if (!strcmp(a, "--synthetic")) o.synthetic = true;
        else if (!strcmp(a, "--vocab")) o.synthetic_vocab = atoi(val());
        else if (!strcmp(a, "--fused")) o.fused = atoi(val());
        else if (!strcmp(a, "--math")) {
            const char *m = val();
            o.math = !strcmp(m, "tf32") ? BMB_MATH_TF32 : (!strcmp(m, "bf16") ? BMB_MATH_BF16 : BMB_MATH_FP32);
        } else if (!strcmp(a, "--gpus")) {
            if (atoi(val()) != 1) { fprintf(stderr, "one GPU per process: launch one process per GPU for data parallelism\n"); return 1; }
        } else { fprintf(stderr, "unknown arg %s\n", a); return 1; }
    }

    // --load: restore a checkpoint and generate; no training, no dataset (src/train_gpt.cu:279-289).
    if (o.load_path) {
        bmb_train_config hc{};
        int nvocab = 0;
        char itos[256];
        CHECK(bmb_checkpoint_header(o.load_path, &hc, &nvocab, itos, 256, nullptr, nullptr));
        bmb_train_config c = make_config(o, hc.max_seq_len, hc.vocab_size, hc.padded_vocab, hc.n_layer, hc.n_head, hc.n_embd);
        CHECK(bmb_trainer_create(&run.t, &c, o.seed));
        CHECK(bmb_trainer_load(run.t, o.load_path, 0, nullptr));
        printf("loaded %s: %d layers, %d heads, %d embd, ctx %d, vocab %d, %.2fM params\n", o.load_path, hc.n_layer, hc.n_head,
               hc.n_embd, hc.max_seq_len, hc.vocab_size, bmb_trainer_num_params(run.t) / 1e6);
        o.T = hc.max_seq_len;
        run.corpus.itos.assign(itos, itos + std::min(nvocab, 256));
        printf("\n%s\n", run.sample(o.sample_len, o.seed + 1).c_str());
        bmb_trainer_destroy(run.t);
        return 0;
    }

    if (o.synthetic) {
        run.V = o.synthetic_vocab;
    } else {
        run.corpus = read_text(o.data_path, 0.1f);
        run.V = (int)run.corpus.itos.size();
        if ((int)run.corpus.train.size() < o.T + 3 || (int)run.corpus.val.size() < o.T + 3) {
            fprintf(stderr, "%s is too short for windows of %d tokens\n", o.data_path, o.T + 1);
            return 1;
        }
    }
    run.Vp = ((run.V + 127) / 128) * 128;       // padded so that the head product is aligned
    if (o.synthetic) printf("data      synthetic token ids uniform over vocab %d (padded %d)\n", run.V, run.Vp);
    else printf("data      %zu train / %zu val tokens, vocab %d (padded %d)\n", run.corpus.train.size(), run.corpus.val.size(), run.V, run.Vp);

    bmb_train_config c = make_config(o, o.T, run.V, run.Vp, o.n_layer, o.n_head, o.n_embd);
    CHECK(bmb_trainer_create(&run.t, &c, o.seed));
    int step0 = 0;
    if (o.resume_path) {
        CHECK(bmb_trainer_load(run.t, o.resume_path, 1, &step0));
        printf("resumed   %s at step %d (parameters, AdamW moments)\n", o.resume_path, step0);
    }
    size_t np = 0, na = 0, ns = 0;
    CHECK(bmb_trainer_memory(run.t, &np, &na, &ns));
    const double param_mb = np * 4.0 / 1048576.0, act_mb = na * 4.0 / 1048576.0, gact_mb = ns * 4.0 / 1048576.0;
    printf("model     %d layers, %d heads, %d embd, ctx %d, %s attention\n", o.n_layer, o.n_head, o.n_embd, o.T, o.use_flash ? "fused" : "unfused");
    printf("params    %.2fM (%.1f MB; +%.1f MB grads, +%.1f MB adam state)\n", np / 1e6, param_mb, param_mb, 2 * param_mb);
    printf("memory    %.1f MB forward activations, %.1f MB backward scratch\n", act_mb, gact_mb);
    printf("total     %.2f GB resident (params+grads+adam+activations+scratch)\n", (4.0 * param_mb + act_mb + gact_mb) / 1024.0);
    if (o.alloc_only) { bmb_trainer_destroy(run.t); return 0; }

    std::mt19937 rng(o.seed);
    std::vector<int> x((size_t)o.B * o.T), y((size_t)o.B * o.T);
    const double tokens_per_step = (double)o.B * o.T;
    const double flops_per_step = 6.0 * tokens_per_step * np + 12.0 * o.n_layer * o.n_head * (double)o.T * o.T * (o.n_embd / o.n_head) * o.B;
    float best_val = 1e30f;
    int best_step = 0;
    const int last = step0 + o.steps;
    for (int step = step0 + 1; step <= last; ++step) {
        run.batch(false, rng, x, y);
        CHECK(bmb_trainer_sync(run.t));
        const auto t0 = std::chrono::steady_clock::now();
        CHECK(bmb_trainer_upload(run.t, x.data(), y.data()));
        const float lr_now = lr_at(step, o.warmup, last, o.lr);
        CHECK(bmb_trainer_step(run.t, lr_now, step));
        const bool report = (step % 10 == 0 || step == step0 + 1);
        float loss = 0.0f, gnorm = 0.0f;
        if (report) {
            CHECK(bmb_trainer_loss(run.t, &loss));           // blocks: the step is over
            CHECK(bmb_trainer_grad_norm(run.t, &gnorm));
        } else {
            CHECK(bmb_trainer_sync(run.t));
        }
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        if (report) {
            printf("step %5d/%d  loss %.4f  lr %.2e  |g| %.3f  %6.1f ms  %7.0f tok/s  %5.0f GFLOP/s\n", step, last, loss, lr_now, gnorm,
                   ms, tokens_per_step / (ms * 1e-3), flops_per_step / (ms * 1e-3) / 1e9);
            fflush(stdout);
        }
        if (o.eval_every > 0 && step % o.eval_every == 0) {
            const float vl = run.evaluate(true, 7777, o.eval_batches);
            const bool best = vl < best_val;
            if (best) {
                best_val = vl;
                best_step = step;
                if (o.save_path && *o.save_path)
                    CHECK(bmb_trainer_save(run.t, o.save_path, run.corpus.itos.data(), (int)run.corpus.itos.size(), o.save_optimizer ? 1 : 0, step));
            }
            printf("  [eval] step %d  val loss %.4f  (%d batches)%s\n", step, vl, o.eval_batches, best ? "  <- best" : "");
            fflush(stdout);
        }
        if (o.sample_every > 0 && step % o.sample_every == 0 && !o.synthetic) {
            printf("  [sample] ------------------------------------------\n%s\n", run.sample(o.sample_len, o.seed + 1 + step).c_str());
            printf("  ---------------------------------------------------\n");
            fflush(stdout);
        }
    }
    const float final_val = run.evaluate(true, 7777, o.eval_batches), final_train = run.evaluate(false, 8888, o.eval_batches);
    printf("\nfinal  train loss %.4f   val loss %.4f   (%d batches each)\n", final_train, final_val, o.eval_batches);
    printf("best   val loss %.4f at step %d (checkpoint saved there)\n", best_val, best_step);
    if (o.sample_len > 0 && !o.synthetic) printf("\nfinal sample:\n%s\n", run.sample(o.sample_len, o.seed + 1).c_str());
    bmb_trainer_destroy(run.t);
    return 0;
}
