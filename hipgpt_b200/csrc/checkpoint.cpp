// Reader of HipGPT's checkpoint and run-configuration files (host code, no CUDA calls).
//
// Checkpoint (GPTModel::save_checkpoint, src/gpt_model.cpp:355-388, with TransformerLayer::save,
// src/transformer_layer.cpp:312-344): raw little-endian values, no magic number and no version:
//     int32 V, S, E, L;  float tok[V][E];  float pos[S][E];
//     L times { int32 E, H, F;  Wqkv[E][3E], Wo[E][E], W1[E][F], W2[F][E], bqkv[3E], bo[E], b1[F], b2[E],
//               attn gamma[E], attn beta[E], ffn gamma[E], ffn beta[E] };
//     float out_proj[E][V].
// Optimiser state is not in the file.  hipgpt_gpt_create wants the same tensors in the same order without
// the integer headers; this file strips them and checks what they say.
// Run configuration (save_config, src/train_gpt.cpp:60-102): a JSON object with "model" {vocab_size,
// max_seq_len, embed_dim, num_heads, ff_hidden_dim, num_layers}, "tokenizer" {path, tokens_path},
// "training" {...}, "checkpoint" {latest, step}; file names inside it are relative to its own directory
// (src/generate.cpp:99-103).  Only the keys named here are read.
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "attn_common.cuh"

namespace hipgpt {
namespace {

struct File {
    FILE *f = nullptr;
    explicit File(const char *path) : f(path ? fopen(path, "rb") : nullptr) {}
    ~File() { if (f) fclose(f); }
};

bool read_i32(FILE *f, int *v, int n) { return fread(v, sizeof(int32_t), (size_t)n, f) == (size_t)n; }

long long per_layer_floats(long long E, long long F) { return E * 3 * E + E * E + E * F + F * E + 3 * E + E + F + E + 4 * E; }

// V, S, E, L from the head of the file and H, F from the first layer's own header.
int read_header(FILE *f, const char *path, int *hdr6)
{
    int h4[4];
    if (!read_i32(f, h4, 4)) return fail(HIPGPT_ERR_BAD_ARG, "%s: shorter than its 16-byte header", path);
    const int V = h4[0], S = h4[1], E = h4[2], L = h4[3];
    if (V <= 0 || S <= 0 || E <= 0 || L <= 0 || V > (1 << 24) || S > (1 << 20) || E > (1 << 16) || L > 4096)
        return fail(HIPGPT_ERR_BAD_ARG, "%s: implausible header V=%d S=%d E=%d L=%d (not a HipGPT checkpoint?)", path, V, S, E, L);
    if (fseek(f, (long)(((long long)V + S) * E * (long long)sizeof(float)), SEEK_CUR) != 0)
        return fail(HIPGPT_ERR_BAD_ARG, "%s: cannot seek past the embeddings", path);
    int l3[3];
    if (!read_i32(f, l3, 3)) return fail(HIPGPT_ERR_BAD_ARG, "%s: ends before the first layer", path);
    if (l3[0] != E || l3[1] <= 0 || l3[2] <= 0 || E % l3[1] != 0)
        return fail(HIPGPT_ERR_BAD_ARG, "%s: first layer says E=%d H=%d F=%d against E=%d in the file header", path, l3[0], l3[1], l3[2], E);
    hdr6[0] = V; hdr6[1] = S; hdr6[2] = E; hdr6[3] = L; hdr6[4] = l3[1]; hdr6[5] = l3[2];
    return HIPGPT_OK;
}

// value of "key" inside the text: an integer, or a string copied to `str`.  The keys this file looks for are
// unique in HipGPT's run configuration except "step" and "path", which it does not read by bare name.
bool json_int(const std::string &text, const char *key, int *out)
{
    const std::string k = std::string("\"") + key + "\"";
    size_t p = text.find(k);
    if (p == std::string::npos) return false;
    p = text.find(':', p + k.size());
    if (p == std::string::npos) return false;
    char *end = nullptr;
    const long v = strtol(text.c_str() + p + 1, &end, 10);
    if (end == text.c_str() + p + 1) return false;
    *out = (int)v;
    return true;
}

bool json_str_after(const std::string &text, const char *section, const char *key, std::string *out)
{
    size_t p = text.find(std::string("\"") + section + "\"");
    if (p == std::string::npos) return false;
    const std::string k = std::string("\"") + key + "\"";
    p = text.find(k, p);
    if (p == std::string::npos) return false;
    p = text.find(':', p + k.size());
    if (p == std::string::npos) return false;
    const size_t a = text.find('"', p + 1);
    if (a == std::string::npos) return false;
    const size_t b = text.find('"', a + 1);
    if (b == std::string::npos) return false;
    *out = text.substr(a + 1, b - a - 1);
    return true;
}

}  // namespace
}  // namespace hipgpt

using namespace hipgpt;

extern "C" {

int hipgpt_checkpoint_header(const char *path, int *V, int *S, int *E, int *L, int *H, int *F)
{
    if (!path || !V || !S || !E || !L || !H || !F) return fail(HIPGPT_ERR_NULL, "path and the six outputs must not be NULL");
    File file(path);
    if (!file.f) return fail(HIPGPT_ERR_BAD_ARG, "cannot open %s", path);
    int h[6];
    const int rc = read_header(file.f, path, h);
    if (rc != HIPGPT_OK) return rc;
    *V = h[0]; *S = h[1]; *E = h[2]; *L = h[3]; *H = h[4]; *F = h[5];
    return HIPGPT_OK;
}

// h_weights receives hipgpt_gpt_weight_count(V, S, E, L, H, F) floats: the file's tensors in order, headers removed.
int hipgpt_checkpoint_weights(const char *path, float *h_weights, long long count)
{
    if (!path || !h_weights) return fail(HIPGPT_ERR_NULL, "path and h_weights must not be NULL");
    File file(path);
    if (!file.f) return fail(HIPGPT_ERR_BAD_ARG, "cannot open %s", path);
    int h[6];
    int rc = read_header(file.f, path, h);
    if (rc != HIPGPT_OK) return rc;
    const long long V = h[0], S = h[1], E = h[2], L = h[3], H = h[4], F = h[5];
    const long long want = (V + S) * E + L * per_layer_floats(E, F) + E * V;
    if (count != want) return fail(HIPGPT_ERR_BAD_ARG, "%s holds %lld floats, the buffer is for %lld", path, want, count);
    if (fseek(file.f, 4 * (long)sizeof(int32_t), SEEK_SET) != 0) return fail(HIPGPT_ERR_BAD_ARG, "%s: cannot rewind", path);
    float *p = h_weights;
    auto take = [&](long long n) { const bool ok = fread(p, sizeof(float), (size_t)n, file.f) == (size_t)n; p += n; return ok; };
    if (!take((V + S) * E)) return fail(HIPGPT_ERR_BAD_ARG, "%s: ends inside the embeddings", path);
    for (long long l = 0; l < L; ++l) {
        int l3[3];
        if (!read_i32(file.f, l3, 3)) return fail(HIPGPT_ERR_BAD_ARG, "%s: ends before layer %lld", path, l);
        if (l3[0] != E || l3[1] != H || l3[2] != F)
            return fail(HIPGPT_ERR_BAD_ARG, "%s: layer %lld says E=%d H=%d F=%d, layer 0 said E=%lld H=%lld F=%lld", path, l, l3[0], l3[1], l3[2], E, H, F);
        if (!take(per_layer_floats(E, F))) return fail(HIPGPT_ERR_BAD_ARG, "%s: ends inside layer %lld", path, l);
    }
    if (!take(E * V)) return fail(HIPGPT_ERR_BAD_ARG, "%s: ends inside the output projection", path);
    if (fgetc(file.f) != EOF) return fail(HIPGPT_ERR_BAD_ARG, "%s: bytes left after the output projection", path);
    return HIPGPT_OK;
}

// The model hyper-parameters and the two file names of a run configuration; names are as stored (relative to
// the configuration's directory).  ckpt_name / tok_name may be NULL.
int hipgpt_run_config(const char *json_path, int *V, int *S, int *E, int *H, int *F, int *L,
                      char *ckpt_name, size_t ckpt_cap, char *tok_name, size_t tok_cap)
{
    if (!json_path || !V || !S || !E || !H || !F || !L) return fail(HIPGPT_ERR_NULL, "path and the six outputs must not be NULL");
    File file(json_path);
    if (!file.f) return fail(HIPGPT_ERR_BAD_ARG, "cannot open %s", json_path);
    std::string text;
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof(buf), file.f)) > 0) text.append(buf, n);
    if (!json_int(text, "vocab_size", V) || !json_int(text, "max_seq_len", S) || !json_int(text, "embed_dim", E) ||
        !json_int(text, "num_heads", H) || !json_int(text, "ff_hidden_dim", F) || !json_int(text, "num_layers", L))
        return fail(HIPGPT_ERR_BAD_ARG, "%s: a key of \"model\" is missing (vocab_size, max_seq_len, embed_dim, num_heads, ff_hidden_dim, num_layers)", json_path);
    std::string s;
    if (ckpt_name && ckpt_cap) {
        if (!json_str_after(text, "checkpoint", "latest", &s)) return fail(HIPGPT_ERR_BAD_ARG, "%s: \"checkpoint\".\"latest\" is missing", json_path);
        snprintf(ckpt_name, ckpt_cap, "%s", s.c_str());
    }
    if (tok_name && tok_cap) {
        if (!json_str_after(text, "tokenizer", "path", &s)) return fail(HIPGPT_ERR_BAD_ARG, "%s: \"tokenizer\".\"path\" is missing", json_path);
        snprintf(tok_name, tok_cap, "%s", s.c_str());
    }
    return HIPGPT_OK;
}

// The generation driver for a checkpoint file: reads the headers, loads the tensors, hands them to hipgpt_gpt_create.
int hipgpt_gpt_create_from_checkpoint(hipgpt_gpt **out, const char *path, int max_batch)
{
    int V, S, E, L, H, F;
    int rc = hipgpt_checkpoint_header(path, &V, &S, &E, &L, &H, &F);
    if (rc != HIPGPT_OK) return rc;
    const long long n = hipgpt_gpt_weight_count(V, S, E, L, H, F);
    std::vector<float> w((size_t)n);
    rc = hipgpt_checkpoint_weights(path, w.data(), n);
    if (rc != HIPGPT_OK) return rc;
    return hipgpt_gpt_create(out, w.data(), V, S, E, L, H, F, max_batch);
}

// The same from a run configuration: the checkpoint it names, next to it; the two must agree on the model.
int hipgpt_gpt_create_from_run(hipgpt_gpt **out, const char *json_path, int max_batch)
{
    int V, S, E, H, F, L;
    char name[512];
    int rc = hipgpt_run_config(json_path, &V, &S, &E, &H, &F, &L, name, sizeof(name), nullptr, 0);
    if (rc != HIPGPT_OK) return rc;
    std::string dir(json_path);
    const size_t slash = dir.find_last_of('/');
    dir = slash == std::string::npos ? std::string() : dir.substr(0, slash + 1);
    const std::string ckpt = dir + name;
    int v2, s2, e2, l2, h2, f2;
    rc = hipgpt_checkpoint_header(ckpt.c_str(), &v2, &s2, &e2, &l2, &h2, &f2);
    if (rc != HIPGPT_OK) return rc;
    if (v2 != V || s2 != S || e2 != E || l2 != L || h2 != H || f2 != F)
        return fail(HIPGPT_ERR_BAD_ARG, "%s describes V=%d S=%d E=%d L=%d H=%d F=%d, %s holds V=%d S=%d E=%d L=%d H=%d F=%d",
                    json_path, V, S, E, L, H, F, ckpt.c_str(), v2, s2, e2, l2, h2, f2);
    return hipgpt_gpt_create_from_checkpoint(out, ckpt.c_str(), max_batch);
}

}  // extern "C"
