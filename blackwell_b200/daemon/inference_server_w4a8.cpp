// JSON-lines inference daemon on the batched decode-step driver (bw_decode_*).
//
// It speaks the protocol of the reference's daemon (server/inference_server_int4_batched.cu:340-384): one request per
// stdin line, {"prompts": ["...", ...], "max_tokens": n, "temperature": t}, one response per stdout line,
// {"tokens": [[...], ...], "text": ["...", ...]}; diagnostics on stderr; "Ready." once the model is loaded.  Where the
// reference generates the prompts of a request one after the other with batch 1 and a host decision per token
// (:355-360, generate_one :237-303), this daemon runs them together: all prompts of a request (in groups of the
// engine's batch) advance one token per replay of the captured decode step, each at its own position; the prompt
// tables, the sampled ids and the generated tokens stay in device memory until the group is finished.  Greedy
// decoding only (the reference's temperature 0 path); like the reference, a sequence yields max_tokens + 1 ids --
// the id sampled at the last prompt position and max_tokens more -- and stops after the end-of-text id 151643.
//
// usage: inference_server_w4a8 [--weights DIR] [--tokenizer FILE] [--batch B] [--max-seq S] [--act-bits 4|8]
// The model shape is read from the weight files (layer count, hidden size, head counts, intermediate size, vocabulary).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <climits>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/blackwell_b200.h"

namespace {

// ------------------------------------------------------------------------------------------------ tokenizer
// Byte-level BPE over the file layout of tokenizer_data.bin (include/blackwell/bpe_tokenizer.h:168-296): header
// {vocab, merges, added}, 256 byte-encoder codepoints, vocab entries {id u32, length u16, bytes}, added tokens
// {id u32, length u16, special u8, bytes}, merges {length u16, left, length u16, right}.
struct Tokenizer {
    std::string byte_str[256];
    std::unordered_map<std::string, uint8_t> str_byte;
    std::unordered_map<std::string, uint32_t> vocab;
    std::unordered_map<uint32_t, std::string> id_str;
    std::unordered_map<std::string, int> merge_rank;

    static std::string utf8(uint32_t cp) {
        std::string s;
        if (cp < 0x80) s += (char)cp;
        else if (cp < 0x800) { s += (char)(0xC0 | (cp >> 6)); s += (char)(0x80 | (cp & 0x3F)); }
        else { s += (char)(0xE0 | (cp >> 12)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
        return s;
    }
    static bool rd(FILE* f, void* p, size_t n) { return fread(p, 1, n, f) == n; }

    bool load(const char* path) {
        FILE* f = fopen(path, "rb");
        if (!f) return false;
        uint32_t nv = 0, nm = 0, na = 0;
        bool ok = rd(f, &nv, 4) && rd(f, &nm, 4) && rd(f, &na, 4);
        for (int i = 0; ok && i < 256; ++i) {
            uint32_t cp = 0;
            ok = rd(f, &cp, 4);
            byte_str[i] = utf8(cp);
            str_byte[byte_str[i]] = (uint8_t)i;
        }
        for (uint32_t i = 0; ok && i < nv; ++i) {
            uint32_t id = 0; uint16_t len = 0;
            ok = rd(f, &id, 4) && rd(f, &len, 2);
            std::string s(len, '\0');
            ok = ok && (len == 0 || rd(f, &s[0], len));
            vocab[s] = id; id_str[id] = s;
        }
        for (uint32_t i = 0; ok && i < na; ++i) {
            uint32_t id = 0; uint16_t len = 0; uint8_t special = 0;
            ok = rd(f, &id, 4) && rd(f, &len, 2) && rd(f, &special, 1);
            std::string s(len, '\0');
            ok = ok && (len == 0 || rd(f, &s[0], len));
            vocab[s] = id; id_str[id] = s;
        }
        for (uint32_t i = 0; ok && i < nm; ++i) {
            uint16_t ll = 0, rl = 0;
            ok = rd(f, &ll, 2);
            std::string l(ll, '\0');
            ok = ok && (ll == 0 || rd(f, &l[0], ll)) && rd(f, &rl, 2);
            std::string r(rl, '\0');
            ok = ok && (rl == 0 || rd(f, &r[0], rl));
            merge_rank[l + " " + r] = (int)i;
        }
        fclose(f);
        return ok;
    }

    // Pre-tokens: an optional leading space glued to a run of letters, a run of digits, a run of other characters, or
    // a run of white space.
    static std::vector<std::string> pretokenize(const std::string& t) {
        auto cls = [](unsigned char c) { return isalpha(c) || c >= 0x80 ? 0 : (isdigit(c) ? 1 : (isspace(c) ? 3 : 2)); };
        std::vector<std::string> out;
        size_t i = 0;
        while (i < t.size()) {
            size_t j = i;
            if (t[i] == ' ' && i + 1 < t.size() && cls((unsigned char)t[i + 1]) != 3) ++j;
            const int c = cls((unsigned char)t[j]);
            size_t k = j;
            while (k < t.size() && cls((unsigned char)t[k]) == c) ++k;
            out.push_back(t.substr(i, k - i));
            i = k;
        }
        return out;
    }

    std::vector<int> encode(const std::string& text) const {
        std::vector<int> ids;
        for (const std::string& chunk : pretokenize(text)) {
            std::string enc;
            for (unsigned char c : chunk) enc += byte_str[c];
            auto whole = vocab.find(enc);
            if (whole != vocab.end()) { ids.push_back((int)whole->second); continue; }
            std::vector<std::string> sym;
            for (size_t i = 0; i < enc.size();) {
                const unsigned char c = enc[i];
                const int n = c >= 0xF0 ? 4 : (c >= 0xE0 ? 3 : (c >= 0xC0 ? 2 : 1));
                sym.push_back(enc.substr(i, n));
                i += n;
            }
            while (sym.size() > 1) {  // merge the adjacent pair of lowest rank until none is left
                int best = INT_MAX, at = -1;
                for (size_t j = 0; j + 1 < sym.size(); ++j) {
                    auto it = merge_rank.find(sym[j] + " " + sym[j + 1]);
                    if (it != merge_rank.end() && it->second < best) { best = it->second; at = (int)j; }
                }
                if (at < 0) break;
                sym[at] += sym[at + 1];
                sym.erase(sym.begin() + at + 1);
            }
            for (const std::string& s : sym) {
                auto it = vocab.find(s);
                if (it != vocab.end()) { ids.push_back((int)it->second); continue; }
                for (unsigned char c : s) {
                    auto b = vocab.find(byte_str[c]);
                    if (b != vocab.end()) ids.push_back((int)b->second);
                }
            }
        }
        return ids;
    }

    std::string decode(int id) const {
        auto it = id_str.find((uint32_t)id);
        if (it == id_str.end()) return "";
        const std::string& s = it->second;
        std::string out;
        for (size_t i = 0; i < s.size();) {
            const unsigned char c = s[i];
            const int n = c >= 0xF0 ? 4 : (c >= 0xE0 ? 3 : (c >= 0xC0 ? 2 : 1));
            auto b = str_byte.find(s.substr(i, n));
            if (b != str_byte.end()) out += (char)b->second;
            else out += s.substr(i, n);
            i += n;
        }
        return out;
    }
};

// ------------------------------------------------------------------------------------------------ tiny JSON helpers
std::vector<std::string> parse_prompts(const std::string& json) {
    std::vector<std::string> out;
    size_t p = json.find("\"prompts\"");
    if (p == std::string::npos) return out;
    p = json.find('[', p);
    if (p == std::string::npos) return out;
    for (++p; p < json.size() && json[p] != ']'; ++p) {
        if (json[p] != '"') continue;
        std::string s;
        for (++p; p < json.size() && json[p] != '"'; ++p) {
            if (json[p] == '\\' && p + 1 < json.size()) {
                ++p;
                s += json[p] == 'n' ? '\n' : (json[p] == 't' ? '\t' : json[p]);
            } else {
                s += json[p];
            }
        }
        out.push_back(s);
    }
    return out;
}
double parse_number(const std::string& json, const char* key, double def) {
    size_t p = json.find(key);
    if (p == std::string::npos) return def;
    p += strlen(key);
    while (p < json.size() && (json[p] == ' ' || json[p] == ':' || json[p] == '"')) ++p;
    return p < json.size() ? strtod(json.c_str() + p, nullptr) : def;
}
std::string json_escape(const std::string& s) {
    std::string r;
    for (unsigned char c : s) {
        if (c == '"') r += "\\\"";
        else if (c == '\\') r += "\\\\";
        else if (c == '\n') r += "\\n";
        else if (c == '\r') r += "\\r";
        else if (c == '\t') r += "\\t";
        else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); r += b; }
        else r += (char)c;
    }
    return r;
}

constexpr int kEos = 151643;

}  // namespace

int main(int argc, char** argv) {
    std::string weights = "weights_int4_qwen3_8b", tok_path = "tokenizer_data.bin";
    int batch = 8, max_seq = 4096, act_bits = 8, max_new_cap = 512;
    for (int i = 1; i + 1 < argc; i += 2) {
        const std::string k = argv[i];
        if (k == "--weights") weights = argv[i + 1];
        else if (k == "--tokenizer") tok_path = argv[i + 1];
        else if (k == "--batch") batch = atoi(argv[i + 1]);
        else if (k == "--max-seq") max_seq = atoi(argv[i + 1]);
        else if (k == "--act-bits") act_bits = atoi(argv[i + 1]);
        else { fprintf(stderr, "unknown option %s\n", k.c_str()); return 2; }
    }
    Tokenizer tok;
    if (!tok.load(tok_path.c_str())) { fprintf(stderr, "FAIL: cannot read %s\n", tok_path.c_str()); return 1; }

    // model shape from the files
    bw_decode_config cfg;
    memset(&cfg, 0, sizeof cfg);
    int K = 0, N = 0;
    if (bw_w4_file_dims((weights + "/0_self_attn.q_proj").c_str(), &K, &N) != 0) { fprintf(stderr, "FAIL: no weights in %s\n", weights.c_str()); return 1; }
    cfg.hidden = K; cfg.n_q_heads = N / 128;
    if (bw_w4_file_dims((weights + "/0_self_attn.k_proj").c_str(), &K, &N) != 0) return 1;
    cfg.n_kv_heads = N / 128;
    if (bw_w4_file_dims((weights + "/0_mlp.gate_proj").c_str(), &K, &N) != 0) return 1;
    cfg.inter = N;
    if (bw_w4_file_dims((weights + "/embed_tokens").c_str(), &K, &N) != 0) return 1;
    cfg.vocab = N;
    int layers = 0;
    while (bw_w4_file_dims((weights + "/" + std::to_string(layers) + "_self_attn.q_proj").c_str(), &K, &N) == 0) ++layers;
    cfg.layers = layers; cfg.head_dim = 128; cfg.eps = 1e-6f; cfg.rope_base = 1000000.0f;
    cfg.batch = batch; cfg.max_seq = max_seq; cfg.max_prompt = max_seq; cfg.max_new = max_new_cap;
    cfg.act_bits = act_bits; cfg.use_graph = 1; cfg.weights_dir = weights.c_str();
    fprintf(stderr, "Loading %d-layer INT4 model (hidden %d, %d/%d heads, inter %d, vocab %d), batch %d, W4A%d...\n", layers,
            cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.inter, cfg.vocab, batch, act_bits);
    bw_decode* eng = nullptr;
    const int ce = bw_decode_create(&cfg, &eng);
    if (ce != 0) { fprintf(stderr, "FAIL: bw_decode_create returned %d\n", ce); return 1; }
    cudaStream_t st;
    if (cudaStreamCreate(&st) != cudaSuccess) return 1;
    fprintf(stderr, "Ready.\n");

    std::string line;
    for (;;) {
        line.clear();
        int c;
        while ((c = getchar()) != EOF && c != '\n') line.push_back((char)c);
        if (c == EOF && line.empty()) break;
        if (line.empty()) continue;
        const int max_tokens = std::min(std::max((int)parse_number(line, "\"max_tokens\"", 30), 1), max_new_cap - 1);
        const double temperature = parse_number(line, "\"temperature\"", 0.0);
        const std::vector<std::string> prompts = parse_prompts(line);
        if (prompts.empty()) { printf("{\"error\":\"no prompts\"}\n"); fflush(stdout); continue; }
        if (temperature >= 0.01) { printf("{\"error\":\"greedy decoding only (temperature 0)\"}\n"); fflush(stdout); continue; }
        std::vector<std::vector<int>> results(prompts.size());
        bool failed = false;
        for (size_t g0 = 0; g0 < prompts.size() && !failed; g0 += batch) {
            const int n = (int)std::min(prompts.size() - g0, (size_t)batch);
            std::vector<std::vector<int>> ids(batch, std::vector<int>(1, 0));  // idle slots run a one-token dummy
            int longest = 1;
            for (int m = 0; m < n; ++m) {
                ids[m] = tok.encode(prompts[g0 + m]);
                if (ids[m].empty()) ids[m].push_back(0);
                if ((int)ids[m].size() > max_seq - max_tokens - 1) ids[m].resize(std::max(1, max_seq - max_tokens - 1));
                longest = std::max(longest, (int)ids[m].size());
            }
            std::vector<int> table((size_t)batch * longest, 0), lens(batch, 1);
            for (int m = 0; m < batch; ++m) {
                lens[m] = (int)ids[m].size();
                std::copy(ids[m].begin(), ids[m].end(), table.begin() + (size_t)m * longest);
            }
            int e = bw_decode_begin(eng, table.data(), lens.data(), longest, st);
            // the longest prompt needs longest + max_tokens steps for its max_tokens + 1 ids
            for (int s = 0; e == 0 && s < longest + max_tokens; ++s) e = bw_decode_step(eng, st);
            std::vector<int> gen((size_t)batch * max_new_cap);
            if (e == 0) e = bw_decode_result(eng, gen.data(), st);
            int status = 0;
            if (e == 0) e = bw_device_status(&status);
            if (e != 0 || status != 0) { fprintf(stderr, "FAIL: decode error %d, device status %d\n", e, status); failed = true; break; }
            for (int m = 0; m < n; ++m)
                for (int j = 0; j <= max_tokens; ++j) {
                    const int id = gen[(size_t)m * max_new_cap + j];
                    if (id < 0) break;
                    results[g0 + m].push_back(id);
                    if (id == kEos) break;
                }
        }
        if (failed) { printf("{\"error\":\"decode failed\"}\n"); fflush(stdout); continue; }
        std::string out = "{\"tokens\":[";
        for (size_t m = 0; m < results.size(); ++m) {
            out += m ? ",[" : "[";
            for (size_t i = 0; i < results[m].size(); ++i) out += (i ? "," : "") + std::to_string(results[m][i]);
            out += "]";
        }
        out += "],\"text\":[";
        for (size_t m = 0; m < results.size(); ++m) {
            std::string text;
            for (int id : results[m]) text += tok.decode(id);
            out += std::string(m ? "," : "") + "\"" + json_escape(text) + "\"";
        }
        out += "]}";
        printf("%s\n", out.c_str());
        fflush(stdout);
    }
    bw_decode_destroy(eng);
    return 0;
}
