// Host runtime of the framework (C++17, no CUDA): random numbers that are bit-identical to
// PyTorch's CPU mt19937 stream, the token-shard data loader with a background prefetch thread, the
// multiple-choice evaluation loader, the tokenizer decoder, the sampler, learning-rate schedules and
// the outlier detector.  Everything is exported through a small C API used from Python via ctypes.
// Errors never terminate the process: functions return a non-zero code and llmc_host_last_error()
// describes what went wrong.
//
// File formats and stream semantics follow the reference so that shards, evaluation files,
// tokenizer files and saved loader states are interchangeable with it:
//   llmc/rand.h, llmc/dataloader.h, llmc/tokenizer.h, llmc/sampler.h, llmc/schedulers.h,
//   llmc/outlier_detector.h of the reference.
#include <fcntl.h>
#include <glob.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

static thread_local std::string g_err;
static int fail(const std::string& msg) { g_err = msg; return -1; }
API const char* llmc_host_last_error() { return g_err.c_str(); }
API int llmc_host_version() { return 1; }

// ---------------------------------------------------------------------------------------------
// mt19937 with the exact output functions PyTorch uses on the CPU

struct MTState {           // 2520 bytes; stored verbatim in optimizer state files
    unsigned long long seed;
    int left;
    unsigned int next;
    unsigned int state[624];
    unsigned int matrix_a[2];
};
static_assert(sizeof(MTState) == 2520, "state layout must stay byte compatible");

static void mt_seed(MTState* s, unsigned int seed) {
    s->seed = seed;
    s->matrix_a[0] = 0u; s->matrix_a[1] = 0x9908b0dfu;
    s->state[0] = seed;
    for (unsigned int j = 1; j < 624; j++) s->state[j] = 1812433253u * (s->state[j - 1] ^ (s->state[j - 1] >> 30)) + j;
    s->left = 1; s->next = 0;
}
static void mt_refill(MTState* s) {
    const unsigned int UP = 0x80000000u, LO = 0x7fffffffu;
    unsigned int* st = s->state;
    for (int j = 0; j < 624; j++) {
        unsigned int y = (st[j] & UP) | (st[(j + 1) % 624] & LO);
        st[j] = st[(j + 397) % 624] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
    }
    s->left = 624; s->next = 0;
}
static unsigned int mt_u32(MTState* s) {
    if (--s->left <= 0) mt_refill(s);
    unsigned int y = s->state[s->next++];
    y ^= y >> 11; y ^= (y << 7) & 0x9d2c5680u; y ^= (y << 15) & 0xefc60000u; y ^= y >> 18;
    return y;
}
static unsigned long long mt_u64(MTState* s) { unsigned long long hi = mt_u32(s); return (hi << 32) | mt_u32(s); }
static float mt_f32(MTState* s) { return (mt_u32(s) & ((1u << 24) - 1)) * (1.0f / (1u << 24)); }
static double mt_f64(MTState* s) { return (mt_u64(s) & ((1ull << 53) - 1)) * (1.0 / (1ull << 53)); }

static void box_muller_16(float* d, float mean, float std) {
    for (int t = 0; t < 8; t++) {
        float u1 = 1 - d[t], u2 = d[t + 8];
        float radius = sqrtf(-2 * logf(u1 + 1e-12f));
        float theta = (float)(2.0 * M_PI * u2);
        d[t] = radius * cosf(theta) * std + mean;
        d[t + 8] = radius * sinf(theta) * std + mean;
    }
}
static void mt_normal(MTState* s, float* d, size_t n, float mean, float std) {
    if (n >= 16) {
        for (size_t t = 0; t < n; t++) d[t] = mt_f32(s);
        for (size_t i = 0; i + 15 < n; i += 16) box_muller_16(d + i, mean, std);
        if (n % 16 != 0) {                       // the ragged tail is redrawn as a full block of 16
            float* tail = d + n - 16;
            for (int i = 0; i < 16; i++) tail[i] = mt_f32(s);
            box_muller_16(tail, mean, std);
        }
    } else {
        double cached = 0.0; bool have = false;
        for (size_t t = 0; t < n; t++) {
            if (have) { d[t] = (float)(cached * std + mean); have = false; continue; }
            float u1 = (float)mt_f64(s), u2 = (float)mt_f64(s);
            float radius = sqrtf(-2 * logf(1 - u2 + 1e-12f));
            float theta = (float)(2.0 * M_PI * u1);
            cached = radius * sinf(theta); have = true;
            d[t] = radius * cosf(theta) * std + mean;
        }
    }
}
static void mt_permute(MTState* s, int* d, int n) {      // Fisher-Yates from the back
    for (int i = n - 1; i > 0; i--) { int j = (int)(mt_u32(s) % (unsigned)(i + 1)); int t = d[i]; d[i] = d[j]; d[j] = t; }
}

API void* llmc_rng_new(unsigned int seed) { MTState* s = new MTState; mt_seed(s, seed); return s; }
API void llmc_rng_free(void* p) { delete (MTState*)p; }
API unsigned int llmc_rng_u32(void* p) { return mt_u32((MTState*)p); }
API float llmc_rng_f32(void* p) { return mt_f32((MTState*)p); }
API void llmc_rng_uniform(void* p, float* out, long long n, float from, float to) {
    for (long long i = 0; i < n; i++) out[i] = mt_f32((MTState*)p) * (to - from) + from;
}
API void llmc_rng_normal(void* p, float* out, long long n, float mean, float std) { mt_normal((MTState*)p, out, (size_t)n, mean, std); }
API void llmc_rng_permutation(void* p, int* data, int n) { mt_permute((MTState*)p, data, n); }
API void llmc_rng_get_state(void* p, void* out) { memcpy(out, p, sizeof(MTState)); }
API void llmc_rng_set_state(void* p, const void* in) { memcpy(p, in, sizeof(MTState)); }

// ---------------------------------------------------------------------------------------------
// token shards: 256 x int32 header {20240520, 1, ntok} then ntok x uint16 (GPT-2 vocabulary), or
// {20240801, 7, ntok} then ntok x uint32 (LLaMA-3 vocabulary, which does not fit 16 bits)

struct Shard {
    std::string path;
    int64_t ntok = 0;
};
struct MappedFile {
    const uint8_t* base = nullptr; size_t size = 0; int fd = -1;
    void close_() { if (base) munmap((void*)base, size); if (fd >= 0) close(fd); base = nullptr; fd = -1; size = 0; }
    int open_(const std::string& path) {
        close_();
        fd = open(path.c_str(), O_RDONLY);
        if (fd < 0) return fail("cannot open " + path);
        struct stat st; if (fstat(fd, &st) != 0) return fail("cannot stat " + path);
        size = (size_t)st.st_size;
        void* m = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
        if (m == MAP_FAILED) { base = nullptr; return fail("cannot map " + path); }
        base = (const uint8_t*)m;
        madvise(m, size, MADV_WILLNEED);
        return 0;
    }
};

static int read_shard_header(const std::string& path, int64_t* ntok, size_t* tok_bytes) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return fail("cannot open " + path);
    int header[256];
    if (fread(header, sizeof(int), 256, f) != 256) { fclose(f); return fail("short header in " + path); }
    fseek(f, 0, SEEK_END); int64_t size = ftell(f); fclose(f);
    if (header[0] == 20240520) {
        if (header[1] != 1) return fail("bad version in token shard " + path);
        *tok_bytes = sizeof(uint16_t);
    } else if (header[0] == 20240801) {
        if (header[1] != 7) return fail("bad version in token shard " + path);
        *tok_bytes = sizeof(uint32_t);
    } else {
        return fail("bad magic in token shard " + path);
    }
    *ntok = header[2];
    if (*ntok <= 0) return fail("empty token shard " + path);
    if (size != (int64_t)(256 * sizeof(int)) + *ntok * (int64_t)*tok_bytes) return fail("size of " + path + " does not match its header");
    return 0;
}

struct DataLoader {
    int rank = 0, nproc = 1, shuffle = 0;
    size_t B = 0, T = 0;
    size_t tok_bytes = sizeof(uint16_t);      // width of a token in the shard files (all shards of a loader agree)
    std::vector<Shard> shards;
    int64_t num_tokens = 0;
    size_t shard_num_samples = 0, current_shard = 0, current_sample = 0;
    MTState rng;
    std::vector<int> shard_indices, intra_indices;
    MappedFile file;
    // prefetch
    std::thread worker; std::mutex mu; std::condition_variable cv;
    bool job_pending = false, job_done = false, quit = false; int job_rc = 0;
    int* job_in = nullptr; int* job_tg = nullptr;

    int load_shard(size_t idx) {
        size_t real = shuffle ? (size_t)shard_indices[idx] : idx;
        if (file.open_(shards[real].path)) return -1;
        size_t total_batch_bytes = (size_t)nproc * B * T * tok_bytes;
        shard_num_samples = ((size_t)shards[real].ntok * tok_bytes - tok_bytes) / total_batch_bytes;
        return 0;
    }
    void prepare_intra() {
        intra_indices.resize(shard_num_samples);
        for (size_t i = 0; i < shard_num_samples; i++) intra_indices[i] = (int)i;
        mt_permute(&rng, intra_indices.data(), (int)shard_num_samples);
    }
    int reset() {
        current_shard = 0; current_sample = 0;
        if (shuffle) mt_permute(&rng, shard_indices.data(), (int)shards.size());
        if (load_shard(0)) return -1;
        if (shuffle) prepare_intra();
        return 0;
    }
    int advance() {
        if (current_shard == shards.size() - 1) return reset();
        current_shard = (current_shard + 1) % shards.size();
        current_sample = 0;
        if (load_shard(current_shard)) return -1;
        if (shuffle) prepare_intra();
        return 0;
    }
    int next(int* inputs, int* targets) {
        if (current_sample >= shard_num_samples) { if (advance()) return -1; }
        size_t idx = shuffle ? (size_t)intra_indices[current_sample] : current_sample;
        size_t total_batch_bytes = (size_t)nproc * B * T * tok_bytes;
        size_t off = 256 * sizeof(int) + idx * total_batch_bytes + (size_t)rank * B * T * tok_bytes;
        size_t need = (B * T + 1) * tok_bytes;
        if (off + need > file.size) return fail("batch reaches past the end of the shard");
        const size_t n = B * T;
        if (tok_bytes == sizeof(uint16_t)) {
            const uint16_t* src = (const uint16_t*)(file.base + off);
            for (size_t i = 0; i < n; i++) { inputs[i] = (int)src[i]; targets[i] = (int)src[i + 1]; }
        } else {
            const uint32_t* src = (const uint32_t*)(file.base + off);
            for (size_t i = 0; i < n; i++) { inputs[i] = (int)src[i]; targets[i] = (int)src[i + 1]; }
        }
        current_sample += 1;
        return 0;
    }
    void worker_loop() {
        std::unique_lock<std::mutex> lk(mu);
        while (true) {
            cv.wait(lk, [&] { return job_pending || quit; });
            if (quit) return;
            int* a = job_in; int* b = job_tg;
            lk.unlock();
            int rc = next(a, b);
            lk.lock();
            job_rc = rc; job_pending = false; job_done = true;
            cv.notify_all();
        }
    }
};

API void* llmc_dl_new(const char* pattern, long long B, long long T, int rank, int nproc, int shuffle) {
    glob_t g;
    if (glob(pattern, 0, nullptr, &g) != 0 || g.gl_pathc == 0) { fail(std::string("no files match ") + pattern); globfree(&g); return nullptr; }
    DataLoader* dl = new DataLoader;
    dl->rank = rank; dl->nproc = nproc; dl->shuffle = shuffle; dl->B = (size_t)B; dl->T = (size_t)T;
    for (size_t i = 0; i < g.gl_pathc; i++) {
        Shard s; s.path = g.gl_pathv[i];
        size_t width = 0;
        if (read_shard_header(s.path, &s.ntok, &width)) { globfree(&g); delete dl; return nullptr; }
        if (i > 0 && width != dl->tok_bytes) { fail("shards of one pattern mix 16-bit and 32-bit tokens"); globfree(&g); delete dl; return nullptr; }
        dl->tok_bytes = width;
        if (s.ntok < (int64_t)((size_t)nproc * B * T + 1)) { fail("shard " + s.path + " holds fewer tokens than one global batch"); globfree(&g); delete dl; return nullptr; }
        dl->num_tokens += s.ntok;
        dl->shards.push_back(s);
    }
    globfree(&g);
    if (shuffle) {
        mt_seed(&dl->rng, 42u + (unsigned)rank);
        dl->shard_indices.resize(dl->shards.size());
        for (size_t i = 0; i < dl->shards.size(); i++) dl->shard_indices[i] = (int)i;
    } else {
        mt_seed(&dl->rng, 42u);
    }
    if (dl->reset()) { delete dl; return nullptr; }
    return dl;
}
API void llmc_dl_free(void* p) {
    DataLoader* dl = (DataLoader*)p;
    if (!dl) return;
    if (dl->worker.joinable()) {
        { std::lock_guard<std::mutex> lk(dl->mu); dl->quit = true; }
        dl->cv.notify_all();
        dl->worker.join();
    }
    dl->file.close_();
    delete dl;
}
API int llmc_dl_next(void* p, int* inputs, int* targets) { return ((DataLoader*)p)->next(inputs, targets); }
API int llmc_dl_reset(void* p) { return ((DataLoader*)p)->reset(); }
API int llmc_dl_resume(void* p, long long shard_idx, long long sample_idx) {
    DataLoader* dl = (DataLoader*)p;
    dl->current_shard = (size_t)shard_idx; dl->current_sample = (size_t)sample_idx;
    return dl->load_shard(dl->current_shard);
}
// asynchronous variant: the next batch is produced by a worker thread into caller-owned (pinned) buffers
API int llmc_dl_prefetch(void* p, int* inputs, int* targets) {
    DataLoader* dl = (DataLoader*)p;
    std::lock_guard<std::mutex> lk(dl->mu);
    if (dl->job_pending) return fail("a prefetch is already in flight");
    if (!dl->worker.joinable()) dl->worker = std::thread([dl] { dl->worker_loop(); });
    dl->job_in = inputs; dl->job_tg = targets; dl->job_pending = true; dl->job_done = false;
    dl->cv.notify_all();
    return 0;
}
API int llmc_dl_wait(void* p) {
    DataLoader* dl = (DataLoader*)p;
    std::unique_lock<std::mutex> lk(dl->mu);
    dl->cv.wait(lk, [&] { return dl->job_done || !dl->job_pending; });
    return dl->job_rc;
}
API long long llmc_dl_get(void* p, int what) {
    DataLoader* dl = (DataLoader*)p;
    switch (what) {
        case 0: return dl->num_tokens;
        case 1: return (long long)dl->shard_num_samples;
        case 2: return (long long)dl->current_shard;
        case 3: return (long long)dl->current_sample;
        case 4: return (long long)dl->shards.size();
        case 5: return (long long)dl->intra_indices.size();
        case 6: return dl->shuffle;
    }
    return -1;
}
// shuffle state export / import (what the optimizer state file stores)
API void llmc_dl_get_shuffle_state(void* p, int* shard_indices, int* intra_indices, void* rng_state) {
    DataLoader* dl = (DataLoader*)p;
    memcpy(shard_indices, dl->shard_indices.data(), dl->shard_indices.size() * sizeof(int));
    memcpy(intra_indices, dl->intra_indices.data(), dl->intra_indices.size() * sizeof(int));
    memcpy(rng_state, &dl->rng, sizeof(MTState));
}
API int llmc_dl_set_shuffle_state(void* p, const int* shard_indices, long long n_shards, const int* intra_indices, long long n_intra, const void* rng_state) {
    DataLoader* dl = (DataLoader*)p;
    if ((size_t)n_shards != dl->shards.size()) return fail("saved loader state has a different number of shards");
    dl->shard_indices.assign(shard_indices, shard_indices + n_shards);
    dl->intra_indices.assign(intra_indices, intra_indices + n_intra);
    memcpy(&dl->rng, rng_state, sizeof(MTState));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// evaluation loader (HellaSwag-style multiple choice): header {20240522, 1, num_examples, longest_example_bytes}

struct EvalLoader {
    int rank = 0, nproc = 1; size_t B = 0, T = 0;
    MappedFile file; size_t cursor = 0;
    int num_examples = 0, num_batches = 0, start = 0, end = 0, current = 0;
    std::vector<int> label;
    static constexpr int NC = 4;

    int reset() {
        int per = (num_examples + nproc - 1) / nproc;
        int fit = (int)(B / NC);
        if (fit == 0) return fail("evaluation needs a batch size of at least 4");
        num_batches = (per + fit - 1) / fit;
        start = per * rank; end = per * (rank + 1); if (end > num_examples) end = num_examples;
        cursor = 256 * sizeof(int);
        for (int i = 0; i < start; i++) {
            const uint16_t* h = (const uint16_t*)(file.base + cursor);
            if (cursor + 6 > file.size || h[0] != 65535 || h[2] != (uint16_t)i) return fail("corrupt evaluation file");
            cursor += h[1];
        }
        current = start;
        return 0;
    }
    int next_batch(int* inputs, int* targets, char* mask) {
        memset(mask, 0, B * T);
        int fit = (int)(B / NC);
        label.assign(fit, -1);
        for (int e = 0; e < fit; e++) {
            if (current >= end) break;
            const uint16_t* h = (const uint16_t*)(file.base + cursor);
            if (cursor + 6 > file.size || h[0] != 65535 || h[2] != (uint16_t)current) return fail("corrupt evaluation file");
            const size_t bytes = h[1];
            if (cursor + bytes > file.size) return fail("evaluation example reaches past the end of the file");
            const uint16_t* buf = h + 3;
            int lab = buf[0], nc = buf[1], ctx = buf[2];
            if (lab < 0 || lab >= NC || nc != NC || ctx <= 0 || ctx >= (int)T) return fail("evaluation example does not fit the loader");
            label[e] = lab;
            const uint16_t* ctx_tok = buf + 3;
            const int row0 = e * NC;
            for (int b = 0; b < NC; b++) for (int i = 0; i < ctx; i++) inputs[(size_t)(row0 + b) * T + i] = ctx_tok[i];
            const uint16_t* it = ctx_tok + ctx;
            for (int c = 0; c < NC; c++) {
                int len = it[0];
                if (len <= 0 || ctx + len >= (int)T) return fail("evaluation completion does not fit the sequence length");
                for (int i = 0; i < len; i++) {
                    size_t row = (size_t)(row0 + c) * T;
                    inputs[row + ctx + i] = it[1 + i];
                    targets[row + ctx + i - 1] = it[1 + i];
                    mask[row + ctx + i - 1] = 1;
                }
                it += 1 + len;
            }
            cursor += bytes;
            current++;
        }
        return 0;
    }
    int stat_losses(const float* losses, const char* mask) {
        int correct = 0, fit = (int)(B / NC);
        for (int e = 0; e < fit; e++) {
            float best = 0.f; int best_i = -1; bool active = false;
            for (int b = 0; b < NC; b++) {
                size_t row = (size_t)(e * NC + b) * T;
                float sum = 0.f; int cnt = 0;
                for (size_t t = 0; t < T; t++) if (mask[row + t] == 1) { active = true; sum += losses[row + t]; cnt++; }
                if (cnt > 0) sum /= cnt;
                if (b == 0 || sum < best) { best = sum; best_i = b; }
            }
            if (active && best_i == label[e]) correct++;
        }
        return correct;
    }
};

API void* llmc_eval_new(const char* path, long long B, long long T, int rank, int nproc) {
    EvalLoader* el = new EvalLoader;
    el->rank = rank; el->nproc = nproc; el->B = (size_t)B; el->T = (size_t)T;
    if (el->file.open_(path)) { delete el; return nullptr; }
    if (el->file.size < 256 * sizeof(int)) { fail("evaluation file too small"); delete el; return nullptr; }
    const int* h = (const int*)el->file.base;
    if (h[0] != 20240522 || h[1] != 1) { fail("bad magic/version in evaluation file"); delete el; return nullptr; }
    el->num_examples = h[2];
    if (el->num_examples < nproc) { fail("fewer evaluation examples than processes"); delete el; return nullptr; }
    if (el->reset()) { delete el; return nullptr; }
    return el;
}
API void llmc_eval_free(void* p) { EvalLoader* el = (EvalLoader*)p; if (el) { el->file.close_(); delete el; } }
API int llmc_eval_reset(void* p) { return ((EvalLoader*)p)->reset(); }
API int llmc_eval_next_batch(void* p, int* inputs, int* targets, char* mask) { return ((EvalLoader*)p)->next_batch(inputs, targets, mask); }
API int llmc_eval_stat_losses(void* p, const float* losses, const char* mask) { return ((EvalLoader*)p)->stat_losses(losses, mask); }
API int llmc_eval_get(void* p, int what) {
    EvalLoader* el = (EvalLoader*)p;
    switch (what) { case 0: return el->num_examples; case 1: return el->num_batches; case 2: return el->start; case 3: return el->end; case 4: return el->current; }
    return -1;
}

// ---------------------------------------------------------------------------------------------
// tokenizer (decode only): header {20240328, version 1|2, vocab, eot}, then per token: u8 length, bytes

struct Tokenizer { std::vector<std::string> table; int eot = 50256; };
API void* llmc_tokenizer_new(const char* path) {
    FILE* f = fopen(path, "rb");
    if (!f) { fail(std::string("cannot open ") + path); return nullptr; }
    unsigned int header[256];
    if (fread(header, sizeof(unsigned int), 256, f) != 256 || header[0] != 20240328) { fclose(f); fail("bad tokenizer file"); return nullptr; }
    Tokenizer* t = new Tokenizer;
    int version = (int)header[1];
    unsigned int vocab = header[2];
    if (version == 1) t->eot = 50256; else if (version == 2) t->eot = (int)header[3]; else { fclose(f); delete t; fail("unknown tokenizer version"); return nullptr; }
    t->table.resize(vocab);
    for (unsigned int i = 0; i < vocab; i++) {
        unsigned char len;
        if (fread(&len, 1, 1, f) != 1) { fclose(f); delete t; fail("truncated tokenizer file"); return nullptr; }
        std::string s(len, '\0');
        if (len && fread(&s[0], 1, len, f) != len) { fclose(f); delete t; fail("truncated tokenizer file"); return nullptr; }
        t->table[i] = s;
    }
    fclose(f);
    return t;
}
API void llmc_tokenizer_free(void* p) { delete (Tokenizer*)p; }
API int llmc_tokenizer_vocab(void* p) { return (int)((Tokenizer*)p)->table.size(); }
API int llmc_tokenizer_eot(void* p) { return ((Tokenizer*)p)->eot; }
// copies the bytes of a token into out (up to cap), returns their number or -1
API int llmc_tokenizer_decode(void* p, unsigned int token, char* out, int cap) {
    Tokenizer* t = (Tokenizer*)p;
    if (token >= t->table.size()) return -1;
    const std::string& s = t->table[token];
    int n = (int)s.size() < cap ? (int)s.size() : cap;
    memcpy(out, s.data(), n);
    return n;
}

// ---------------------------------------------------------------------------------------------
// sampler: xorshift* stream and inverse-CDF sampling from logits

API unsigned int llmc_random_u32(unsigned long long* state) {
    *state ^= *state >> 12; *state ^= *state << 25; *state ^= *state >> 27;
    return (unsigned int)((*state * 0x2545F4914F6CDD1Dull) >> 32);
}
API float llmc_random_f32(unsigned long long* state) { return (llmc_random_u32(state) >> 8) / 16777216.0f; }
API int llmc_sample_softmax(const float* logits, int n, float coin) {
    double norm = 0;
    for (int i = 0; i < n; i++) norm += expf(logits[i]);
    coin *= (float)norm;          // compare against unnormalised masses instead of dividing every term
    float cdf = 0.f;
    for (int i = 0; i < n; i++) { cdf += expf(logits[i]); if (coin < cdf) return i; }
    return n - 1;
}

// ---------------------------------------------------------------------------------------------
// learning-rate schedules: 0 cosine, 1 linear, 2 constant, 3 wsd

API float llmc_learning_rate(int type, int step, float lr, int warmup, int train_steps, float final_frac) {
    if (type == 2) return lr;
    if (type == 0) {
        if (step < warmup) return lr * (float)(step + 1) / warmup;
        float ratio = (float)(step - warmup) / (float)(train_steps - warmup);
        float coeff = 0.5f * (1.0f + cosf((float)M_PI * ratio));
        float min_lr = lr * final_frac;
        return min_lr + coeff * (lr - min_lr);
    }
    if (type == 1) {
        if (step < warmup) return lr * (float)(step + 1) / warmup;
        float ratio = (float)(step - warmup) / (float)(train_steps - warmup);
        float min_lr = lr * final_frac;
        return lr - ratio * (lr - min_lr);
    }
    if (type == 3) {   // warmup - stable - (1 - sqrt) decay over the last fifth
        int decay_point = (int)(0.8f * train_steps);
        if (step < warmup) return lr * (float)(step + 1) / warmup;
        if (step < decay_point) return lr;
        float ratio = (float)(step - decay_point) / (float)(train_steps - decay_point);
        if (ratio < 0) ratio = 0; if (ratio > 1) ratio = 1;
        float min_lr = lr * final_frac;
        return min_lr + (1.0f - sqrtf(ratio)) * (lr - min_lr);
    }
    return lr;
}

// ---------------------------------------------------------------------------------------------
// outlier detector: z-score of a new value against a sliding window of 128, in double precision

struct Outlier { int count = 0, index = 0; double buf[128]; double sum = 0, sum_sq = 0; };
API void* llmc_outlier_new() { Outlier* o = new Outlier; memset(o->buf, 0, sizeof(o->buf)); return o; }
API void llmc_outlier_free(void* p) { delete (Outlier*)p; }
API double llmc_outlier_update(void* p, double v) {
    Outlier* o = (Outlier*)p;
    const int W = 128;
    if (o->count < W) {
        o->buf[o->count] = v; o->sum += v; o->sum_sq += v * v; o->count++;
        return NAN;                                  // still filling the window
    }
    o->sum -= o->buf[o->index]; o->sum_sq -= o->buf[o->index] * o->buf[o->index];
    o->buf[o->index] = v; o->sum += v; o->sum_sq += v * v;
    o->index = (o->index + 1) % W;
    double mean = o->sum / W, var = o->sum_sq / W - mean * mean, sd = sqrt(var);
    if (sd == 0.0) return 0.0;
    return (v - mean) / sd;
}

// ---------------------------------------------------------------------------------------------
// CPU matmul out[BT, OC] = inp[BT, C] * weight[OC, C]^T (+ bias): the straightforward loop nest and a register-tiled one, both
// split over threads by rows, for the CPU micro-benchmark (the role of dev/cpu/matmul_forward.c in the reference).

static void split_rows(int rows, int nthreads, const std::function<void(int, int)>& body) {
    if (nthreads < 1) nthreads = 1;
    if (nthreads == 1 || rows < 2 * nthreads) { body(0, rows); return; }
    std::vector<std::thread> pool;
    const int per = (rows + nthreads - 1) / nthreads;
    for (int t = 0; t < nthreads; t++) {
        const int lo = t * per, hi = lo + per < rows ? lo + per : rows;
        if (lo < hi) pool.emplace_back(body, lo, hi);
    }
    for (auto& th : pool) th.join();
}

API void llmc_cpu_matmul_naive(float* out, const float* inp, const float* weight, const float* bias, int BT, int C, int OC, int nthreads) {
    split_rows(BT, nthreads, [&](int lo, int hi) {
        for (int r = lo; r < hi; r++) {
            const float* x = inp + (size_t)r * C;
            for (int o = 0; o < OC; o++) {
                const float* w = weight + (size_t)o * C;
                float acc = bias ? bias[o] : 0.0f;
                for (int c = 0; c < C; c++) acc += x[c] * w[c];
                out[(size_t)r * OC + o] = acc;
            }
        }
    });
}

// Eight input rows share every weight row that is streamed in: eight accumulators live in registers, so the weight matrix is read
// once per eight rows instead of once per row.
API void llmc_cpu_matmul_tiled(float* out, const float* inp, const float* weight, const float* bias, int BT, int C, int OC, int nthreads) {
    constexpr int R = 8;
    split_rows((BT + R - 1) / R, nthreads, [&](int lo, int hi) {
        for (int blk = lo; blk < hi; blk++) {
            const int r0 = blk * R, nr = r0 + R <= BT ? R : BT - r0;
            for (int o = 0; o < OC; o++) {
                const float* w = weight + (size_t)o * C;
                float acc[R];
                for (int k = 0; k < R; k++) acc[k] = bias ? bias[o] : 0.0f;
                if (nr == R) {
                    for (int c = 0; c < C; c++) {
                        const float wv = w[c];
                        for (int k = 0; k < R; k++) acc[k] += inp[(size_t)(r0 + k) * C + c] * wv;
                    }
                } else {
                    for (int c = 0; c < C; c++)
                        for (int k = 0; k < nr; k++) acc[k] += inp[(size_t)(r0 + k) * C + c] * w[c];
                }
                for (int k = 0; k < nr; k++) out[(size_t)(r0 + k) * OC + o] = acc[k];
            }
        }
    });
}
