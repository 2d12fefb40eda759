// A second plain implementation of the Qwen3 dense decoder, in C++ and double precision, written from the
// reference's formulas independently of tests/plain_qwen3.py (loops over scalars instead of tensor algebra; it
// shares no code with that file or with the package). The two must agree to rounding: a misreading of the
// formulas that both share would have to be made twice in two different shapes.
//
//   plain_qwen3 MANIFEST TOKENS OUT
//
// MANIFEST is a text file: first line "config" followed by key=value pairs (layers hidden heads kv_heads head_dim
// inter vocab theta eps tied bias), then "windows w0 w1 ...", "no_rope r0 r1 ...", then one line per tensor:
// "tensor NAME OFFSET COUNT" into the float64 little-endian blob MANIFEST.bin. TOKENS is a text file of token ids.
// OUT receives the logits [tokens, vocab] as float64.
//
// Formulas (paths within mashriram/llm-rs):
//   embedding      llm-core/src/graph/builder.rs:8-14, llm-core/src/backends/candle.rs:1238-1261
//   RMSNorm        llm-core/src/backends/attention.rs:55-68,98-104 (x / sqrt(mean(x^2) + eps) * w)
//   projections    llm-core/src/backends/candle.rs:1276-1340 (W stored [out, in], bias added after)
//   q/k head norm  llm-core/src/graph/builder.rs:123-153 (before the rotation; eps = rms_norm_eps here)
//   rotation       angles pos * theta^(-2i/d), llm-core/src/backends/attention.rs:178-214; pairs (i, i + d/2)
//   attention      llm-core/src/backends/candle.rs:1587-1640, head sharing attention.rs:240-248
//   SwiGLU         llm-core/src/graph/builder.rs:256-297, candle.rs:1645-1663
//   block          builder.rs:74-88,223-254,322-333; head builder.rs:408-437, tied: weights.rs:144-157
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

typedef std::vector<double> Vec;

struct Model {
    std::map<std::string, double> cfg;
    std::vector<int> windows, no_rope;
    std::map<std::string, std::pair<size_t, size_t>> where;
    Vec blob;
    const double* t(const std::string& name) const {
        auto it = where.find(name);
        if (it == where.end()) { std::cerr << "missing tensor " << name << "\n"; std::exit(2); }
        return blob.data() + it->second.first;
    }
    bool has(const std::string& name) const { return where.count(name) != 0; }
    int i(const char* k) const { return (int)cfg.at(k); }
};

static void rms_norm(const double* x, const double* w, int n, double eps, double* out) {
    double ss = 0;
    for (int j = 0; j < n; ++j) ss += x[j] * x[j];
    const double inv = 1.0 / std::sqrt(ss / n + eps);
    for (int j = 0; j < n; ++j) out[j] = x[j] * inv * w[j];
}

// y[t, o] = sum_i x[t, i] W[o, i] (+ b[o])
static Vec linear(const Vec& x, int T, int in, const double* W, int out, const double* b) {
    Vec y((size_t)T * out);
    for (int t = 0; t < T; ++t)
        for (int o = 0; o < out; ++o) {
            double acc = 0;
            const double* xr = &x[(size_t)t * in];
            const double* wr = W + (size_t)o * in;
            for (int k = 0; k < in; ++k) acc += xr[k] * wr[k];
            y[(size_t)t * out + o] = acc + (b ? b[o] : 0.0);
        }
    return y;
}

int main(int argc, char** argv) {
    if (argc != 4) { std::cerr << "usage: plain_qwen3 MANIFEST TOKENS OUT\n"; return 1; }
    Model m;
    {
        std::ifstream f(argv[1]);
        std::string line;
        while (std::getline(f, line)) {
            std::istringstream ss(line);
            std::string kind;
            ss >> kind;
            if (kind == "config") {
                std::string kv;
                while (ss >> kv) { size_t eq = kv.find('='); m.cfg[kv.substr(0, eq)] = std::stod(kv.substr(eq + 1)); }
            } else if (kind == "windows") { int v; while (ss >> v) m.windows.push_back(v);
            } else if (kind == "no_rope") { int v; while (ss >> v) m.no_rope.push_back(v);
            } else if (kind == "tensor") { std::string name; size_t off, n; ss >> name >> off >> n; m.where[name] = {off, n}; }
        }
        std::ifstream b(std::string(argv[1]) + ".bin", std::ios::binary | std::ios::ate);
        const size_t bytes = (size_t)b.tellg();
        b.seekg(0);
        m.blob.resize(bytes / 8);
        b.read(reinterpret_cast<char*>(m.blob.data()), bytes);
    }
    std::vector<int> ids;
    { std::ifstream f(argv[2]); int v; while (f >> v) ids.push_back(v); }
    const int T = (int)ids.size(), L = m.i("layers"), H = m.i("hidden"), nq = m.i("heads"), nkv = m.i("kv_heads"),
              d = m.i("head_dim"), I = m.i("inter"), V = m.i("vocab");
    const double theta = m.cfg.at("theta"), eps = m.cfg.at("eps");
    const bool tied = m.i("tied") != 0, bias = m.i("bias") != 0;
    const int G = nq / nkv, half = d / 2;

    Vec h((size_t)T * H);
    const double* E = m.t("model.embed_tokens.weight");
    for (int t = 0; t < T; ++t)
        for (int j = 0; j < H; ++j) h[(size_t)t * H + j] = E[(size_t)ids[t] * H + j];

    for (int l = 0; l < L; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        auto B = [&](const std::string& n) -> const double* { return bias && m.has(n) ? m.t(n) : nullptr; };
        Vec x((size_t)T * H);
        for (int t = 0; t < T; ++t) rms_norm(&h[(size_t)t * H], m.t(p + "input_layernorm.weight"), H, eps, &x[(size_t)t * H]);
        Vec q = linear(x, T, H, m.t(p + "self_attn.q_proj.weight"), nq * d, B(p + "self_attn.q_proj.bias"));
        Vec k = linear(x, T, H, m.t(p + "self_attn.k_proj.weight"), nkv * d, B(p + "self_attn.k_proj.bias"));
        Vec v = linear(x, T, H, m.t(p + "self_attn.v_proj.weight"), nkv * d, B(p + "self_attn.v_proj.bias"));
        // per-head norm, then the rotation of pairs (i, i + d/2) by pos * theta^(-2i/d)
        auto norm_rotate = [&](Vec& a, int heads, const double* w) {
            Vec tmp(d);
            for (int t = 0; t < T; ++t)
                for (int hd = 0; hd < heads; ++hd) {
                    double* row = &a[((size_t)t * heads + hd) * d];
                    rms_norm(row, w, d, eps, tmp.data());
                    if (m.no_rope[l]) { for (int j = 0; j < d; ++j) row[j] = tmp[j]; continue; }
                    for (int i = 0; i < half; ++i) {
                        const double ang = (double)t * std::pow(theta, -2.0 * i / d);
                        const double c = std::cos(ang), s = std::sin(ang);
                        row[i] = tmp[i] * c - tmp[i + half] * s;
                        row[i + half] = tmp[i + half] * c + tmp[i] * s;
                    }
                }
        };
        norm_rotate(q, nq, m.t(p + "self_attn.q_norm.weight"));
        norm_rotate(k, nkv, m.t(p + "self_attn.k_norm.weight"));
        // causal attention, query head hq reads key head hq / G; a window w > 0 hides keys <= t - w
        Vec o((size_t)T * nq * d, 0.0);
        const int window = m.windows[l];
        const double scale = 1.0 / std::sqrt((double)d);
        Vec sc(T);
        for (int t = 0; t < T; ++t)
            for (int hq = 0; hq < nq; ++hq) {
                const int hk = hq / G;
                const int first = window > 0 ? std::max(0, t - window + 1) : 0;
                double mx = -1e300;
                for (int s = first; s <= t; ++s) {
                    double acc = 0;
                    for (int j = 0; j < d; ++j) acc += q[((size_t)t * nq + hq) * d + j] * k[((size_t)s * nkv + hk) * d + j];
                    sc[s] = acc * scale;
                    mx = std::max(mx, sc[s]);
                }
                double sum = 0;
                for (int s = first; s <= t; ++s) { sc[s] = std::exp(sc[s] - mx); sum += sc[s]; }
                for (int s = first; s <= t; ++s) {
                    const double pr = sc[s] / sum;
                    for (int j = 0; j < d; ++j) o[((size_t)t * nq + hq) * d + j] += pr * v[((size_t)s * nkv + hk) * d + j];
                }
            }
        Vec a = linear(o, T, nq * d, m.t(p + "self_attn.o_proj.weight"), H, B(p + "self_attn.o_proj.bias"));
        for (size_t j = 0; j < h.size(); ++j) h[j] += a[j];
        for (int t = 0; t < T; ++t) rms_norm(&h[(size_t)t * H], m.t(p + "post_attention_layernorm.weight"), H, eps, &x[(size_t)t * H]);
        Vec g = linear(x, T, H, m.t(p + "mlp.gate_proj.weight"), I, nullptr);
        Vec u = linear(x, T, H, m.t(p + "mlp.up_proj.weight"), I, nullptr);
        for (size_t j = 0; j < g.size(); ++j) g[j] = g[j] / (1.0 + std::exp(-g[j])) * u[j];
        Vec y = linear(g, T, I, m.t(p + "mlp.down_proj.weight"), H, nullptr);
        for (size_t j = 0; j < h.size(); ++j) h[j] += y[j];
    }
    Vec f((size_t)T * H);
    for (int t = 0; t < T; ++t) rms_norm(&h[(size_t)t * H], m.t("model.norm.weight"), H, eps, &f[(size_t)t * H]);
    Vec logits = linear(f, T, H, tied ? E : m.t("lm_head.weight"), V, nullptr);
    std::ofstream out(argv[3], std::ios::binary);
    out.write(reinterpret_cast<const char*>(logits.data()), logits.size() * 8);
    return 0;
}
