// A second, scalar statement of the GPT-2 forward pass, independent of tests/plain_gpt2.py:
// another language, its own readers of config.json and model.safetensors, one loop per sum,
// double precision throughout.  The test-suite runs it on tiny random models and compares
// every logit with the plain implementation's float64 run; two implementations written
// apart agree only if both read the formulas the same way (column order of the fused QKV
// matrix, Conv1D [in, out] layout, biased variance, where the scale and the 1/(layer+1)
// factor go, which GELU, n_inner null -> 4 * n_embd, the tied head).
//
// It rests on the reference's formulas, not on running it (the reference is Clojure on the
// JVM over an external library): dev/examples/gpt2.clj:49-62 (embedding + position),
// :139-166 (block: LN -> attention -> add -> LN -> MLP -> add), :176-217 (config keys,
// tensor names, n_inner default), :186-194 (QKV split), :27-36 (Conv1D layout), :108-122
// (tied head), src/pretrained/asr/moonshine.clj:87-108 (LayerNorm and erf-GELU formulas),
// src/pretrained/decoder.clj:56 (1/sqrt(head_dim)).
//
//   scalar_gpt2 MODEL_DIR OUT_FILE id0 id1 id2 ...
// writes logits [T, vocab] as little-endian float64.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

using std::string;
using std::vector;

static string read_file(const string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

// ---- the little JSON that config.json and a safetensors header need
struct Json {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0;
    string str;
    vector<Json> arr;
    vector<std::pair<string, Json>> obj;
    const Json* get(const string& key) const {
        for (auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
};

struct Parser {
    const string& s;
    size_t i = 0;
    explicit Parser(const string& text) : s(text) {}
    void ws() { while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; }
    string str() {
        string out;
        ++i;                                            // opening quote
        while (s.at(i) != '"') {
            if (s[i] == '\\') { ++i; out += s.at(i); } else out += s[i];
            ++i;
        }
        ++i;
        return out;
    }
    Json value() {
        ws();
        Json j;
        char c = s.at(i);
        if (c == '{') {
            j.kind = Json::Obj;
            ++i; ws();
            if (s.at(i) == '}') { ++i; return j; }
            for (;;) {
                ws();
                string key = str();
                ws();
                if (s.at(i) != ':') throw std::runtime_error("json: ':' expected");
                ++i;
                j.obj.emplace_back(key, value());
                ws();
                if (s.at(i) == ',') { ++i; continue; }
                if (s.at(i) == '}') { ++i; break; }
                throw std::runtime_error("json: ',' or '}' expected");
            }
        } else if (c == '[') {
            j.kind = Json::Arr;
            ++i; ws();
            if (s.at(i) == ']') { ++i; return j; }
            for (;;) {
                j.arr.push_back(value());
                ws();
                if (s.at(i) == ',') { ++i; continue; }
                if (s.at(i) == ']') { ++i; break; }
                throw std::runtime_error("json: ',' or ']' expected");
            }
        } else if (c == '"') {
            j.kind = Json::Str;
            j.str = str();
        } else if (s.compare(i, 4, "true") == 0) { j.kind = Json::Bool; j.b = true; i += 4; }
        else if (s.compare(i, 5, "false") == 0) { j.kind = Json::Bool; j.b = false; i += 5; }
        else if (s.compare(i, 4, "null") == 0) { j.kind = Json::Null; i += 4; }
        else {
            size_t used = 0;
            j.kind = Json::Num;
            j.num = std::stod(s.substr(i), &used);
            i += used;
        }
        return j;
    }
};

// ---- tensors by name, widened to double
struct Tensor {
    vector<long> shape;
    vector<double> v;
    double at(long r, long c) const { return v[(size_t)r * shape[1] + c]; }
};

static std::map<string, Tensor> read_safetensors(const string& path) {
    string raw = read_file(path);
    uint64_t n = 0;
    memcpy(&n, raw.data(), 8);                           // little-endian header length
    string header = raw.substr(8, n);
    Json root = Parser(header).value();
    const char* data = raw.data() + 8 + n;
    std::map<string, Tensor> out;
    for (auto& kv : root.obj) {
        if (kv.first == "__metadata__") continue;
        const Json& t = kv.second;
        string name = kv.first;
        if (name.rfind("transformer.", 0) == 0) name = name.substr(12);
        Tensor ten;
        size_t count = 1;
        for (auto& d : t.get("shape")->arr) { ten.shape.push_back((long)d.num); count *= (size_t)d.num; }
        size_t begin = (size_t)t.get("data_offsets")->arr[0].num;
        const string& dt = t.get("dtype")->str;
        ten.v.resize(count);
        for (size_t k = 0; k < count; ++k) {
            if (dt == "F32") {
                float f; memcpy(&f, data + begin + 4 * k, 4); ten.v[k] = f;
            } else if (dt == "BF16") {                   // the upper half of a float32
                uint16_t h; memcpy(&h, data + begin + 2 * k, 2);
                uint32_t bits = (uint32_t)h << 16; float f; memcpy(&f, &bits, 4); ten.v[k] = f;
            } else if (dt == "F64") {
                double f; memcpy(&f, data + begin + 8 * k, 8); ten.v[k] = f;
            } else throw std::runtime_error("unsupported dtype " + dt);
        }
        out[name] = ten;
    }
    return out;
}

// ---- the parts
typedef vector<vector<double>> Rows;

static Rows layer_norm(const Rows& x, const Tensor& gamma, const Tensor& beta, double eps) {
    Rows out(x.size());
    for (size_t r = 0; r < x.size(); ++r) {
        const size_t d = x[r].size();
        double mean = 0;
        for (double v : x[r]) mean += v;
        mean /= d;
        double var = 0;
        for (double v : x[r]) var += (v - mean) * (v - mean);
        var /= d;                                        // biased
        const double inv = 1.0 / std::sqrt(var + eps);
        out[r].resize(d);
        for (size_t c = 0; c < d; ++c) out[r][c] = (x[r][c] - mean) * inv * gamma.v[c] + beta.v[c];
    }
    return out;
}

// y = x . W + b with W stored [in, out]
static Rows conv1d(const Rows& x, const Tensor& w, const Tensor& b) {
    const long n_in = w.shape[0], n_out = w.shape[1];
    Rows out(x.size(), vector<double>(n_out));
    for (size_t r = 0; r < x.size(); ++r)
        for (long o = 0; o < n_out; ++o) {
            double acc = 0;
            for (long i = 0; i < n_in; ++i) acc += x[r][i] * w.at(i, o);
            out[r][o] = acc + b.v[o];
        }
    return out;
}

static double activate(const string& name, double u) {
    if (name == "gelu_new" || name == "gelu_pytorch_tanh")
        return 0.5 * u * (1.0 + std::tanh(std::sqrt(2.0 / M_PI) * (u + 0.044715 * u * u * u)));
    if (name == "gelu") return 0.5 * u * (1.0 + std::erf(u / std::sqrt(2.0)));
    if (name == "relu") return u > 0 ? u : 0;
    throw std::runtime_error("unknown activation " + name);
}

int main(int argc, char** argv) {
    try {
        if (argc < 4) { fprintf(stderr, "usage: scalar_gpt2 MODEL_DIR OUT_FILE ids...\n"); return 2; }
        const string dir = argv[1];
        vector<long> ids;
        for (int a = 3; a < argc; ++a) ids.push_back(atol(argv[a]));
        Json cfg = Parser(read_file(dir + "/config.json")).value();
        auto num = [&](const char* key, double fallback) {
            const Json* j = cfg.get(key);
            return (j && j->kind == Json::Num) ? j->num : fallback;
        };
        auto flag = [&](const char* key, bool fallback) {
            const Json* j = cfg.get(key);
            return (j && j->kind == Json::Bool) ? j->b : fallback;
        };
        const long d = (long)num("n_embd", 0), layers = (long)num("n_layer", 0), heads = (long)num("n_head", 0);
        const long positions = (long)num("n_positions", 0);
        const double eps = num("layer_norm_epsilon", 1e-5);
        const Json* act_j = cfg.get("activation_function");
        const string act = (act_j && act_j->kind == Json::Str) ? act_j->str : "gelu_new";
        const bool scale_w = flag("scale_attn_weights", true);
        const bool scale_layer = flag("scale_attn_by_inverse_layer_idx", false);
        const long dh = d / heads;
        auto w = read_safetensors(dir + "/model.safetensors");
        const long T = (long)ids.size();
        if (T > positions) throw std::runtime_error("sequence longer than n_positions");

        Rows x(T, vector<double>(d));
        for (long t = 0; t < T; ++t)
            for (long c = 0; c < d; ++c) x[t][c] = w["wte.weight"].at(ids[t], c) + w["wpe.weight"].at(t, c);

        for (long l = 0; l < layers; ++l) {
            const string p = "h." + std::to_string(l) + ".";
            Rows h = layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], eps);
            Rows qkv = conv1d(h, w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"]);
            double scale = 1.0;
            if (scale_w) scale /= std::sqrt((double)dh);
            if (scale_layer) scale /= (double)(l + 1);
            Rows mixed(T, vector<double>(d, 0.0));
            for (long hd = 0; hd < heads; ++hd)
                for (long i = 0; i < T; ++i) {
                    vector<double> s(i + 1);
                    double mx = -INFINITY;
                    for (long j = 0; j <= i; ++j) {              // causal: keys j <= i
                        double acc = 0;
                        for (long c = 0; c < dh; ++c)
                            acc += qkv[i][hd * dh + c] * qkv[j][d + hd * dh + c];
                        s[j] = acc * scale;
                        if (s[j] > mx) mx = s[j];
                    }
                    double sum = 0;
                    for (long j = 0; j <= i; ++j) { s[j] = std::exp(s[j] - mx); sum += s[j]; }
                    for (long c = 0; c < dh; ++c) {
                        double acc = 0;
                        for (long j = 0; j <= i; ++j) acc += s[j] / sum * qkv[j][2 * d + hd * dh + c];
                        mixed[i][hd * dh + c] = acc;
                    }
                }
            Rows a = conv1d(mixed, w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"]);
            for (long t = 0; t < T; ++t)
                for (long c = 0; c < d; ++c) x[t][c] += a[t][c];
            Rows h2 = layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], eps);
            Rows u = conv1d(h2, w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"]);
            for (auto& row : u)
                for (double& v : row) v = activate(act, v);
            Rows m = conv1d(u, w[p + "mlp.c_proj.weight"], w[p + "mlp.c_proj.bias"]);
            for (long t = 0; t < T; ++t)
                for (long c = 0; c < d; ++c) x[t][c] += m[t][c];
        }
        Rows hf = layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], eps);
        const Tensor& wte = w["wte.weight"];
        const long vocab = wte.shape[0];
        vector<double> logits((size_t)T * vocab);
        for (long t = 0; t < T; ++t)
            for (long v = 0; v < vocab; ++v) {
                double acc = 0;
                for (long c = 0; c < d; ++c) acc += hf[t][c] * wte.at(v, c);   // tied head, no bias
                logits[(size_t)t * vocab + v] = acc;
            }
        FILE* f = fopen(argv[2], "wb");
        if (!f) throw std::runtime_error("cannot write output");
        fwrite(logits.data(), sizeof(double), logits.size(), f);
        fclose(f);
        return 0;
    } catch (const std::exception& e) {
        fprintf(stderr, "scalar_gpt2: %s\n", e.what());
        return 1;
    }
}
