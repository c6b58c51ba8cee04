// A second plain Llama, in scalar C++: one token at a time, keys and values kept as they arrive, every sum a
// plain loop in double precision.  It exists to be held against tests/plain/llama.py (whole sequences, torch
// tensor operations): two implementations written apart from the same formulas of Leikoe/tesseract, in two
// languages and two shapes (token by token with a growing key/value list here, whole-sequence matrices there).
// A slip in one of them (a transposed weight, the wrong half rotated, a mask off by one, a norm that forgets
// eps) shows as a difference.  It shares no code with the engine or with the other plain model.
//
//   llama_scalar MODEL.bin LOGITS.bin
//
// MODEL.bin (little endian), written by tests/test_plain.py:
//   int32  layers, hidden, heads, kv_heads, head_dim, intermediate, vocab, tied, scaled, original_positions, tokens
//   double eps, theta, factor, low_freq_factor, high_freq_factor
//   int32  token ids [tokens]
//   float  embedding [vocab][hidden]
//   per layer: float input_norm[hidden], q[heads*head_dim][hidden], k[kv*head_dim][hidden], v[kv*head_dim][hidden],
//              o[hidden][heads*head_dim], post_norm[hidden], gate[inter][hidden], up[inter][hidden], down[hidden][inter]
//   float  final_norm[hidden];  float lm_head[vocab][hidden] unless tied
// LOGITS.bin: double [tokens][vocab].
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

namespace {

struct Reader {
    FILE* f;
    template <typename T>
    T one() {
        T v;
        if (fread(&v, sizeof(T), 1, f) != 1) {
            fprintf(stderr, "llama_scalar: short read\n");
            exit(2);
        }
        return v;
    }
    std::vector<double> floats(size_t n) {
        std::vector<float> raw(n);
        if (n && fread(raw.data(), sizeof(float), n, f) != n) {
            fprintf(stderr, "llama_scalar: short read\n");
            exit(2);
        }
        return std::vector<double>(raw.begin(), raw.end());
    }
};

// y[o] = sum_i w[o][i] * x[i]   (a weight is stored [out][in]: y = x W^T, src/cuda/cublas.rs:60-91)
std::vector<double> times_transposed(const std::vector<double>& w, const std::vector<double>& x, int out, int in) {
    std::vector<double> y(out, 0.0);
    for (int o = 0; o < out; ++o) {
        double sum = 0.0;
        for (int i = 0; i < in; ++i) sum += w[(size_t)o * in + i] * x[i];
        y[o] = sum;
    }
    return y;
}

// y = x * rsqrt(mean(x^2) + eps) * weight   (src/cuda/kernels.rs:26-57)
std::vector<double> rms_norm(const std::vector<double>& x, const std::vector<double>& weight, double eps) {
    double squares = 0.0;
    for (double v : x) squares += v * v;
    const double inv = 1.0 / std::sqrt(squares / (double)x.size() + eps);
    std::vector<double> y(x.size());
    for (size_t i = 0; i < x.size(); ++i) y[i] = x[i] * inv * weight[i];
    return y;
}

struct Layer {
    std::vector<double> input_norm, q, k, v, o, post_norm, gate, up, down;
    std::vector<std::vector<double>> keys, values;      // one entry per token seen so far, [kv_heads * head_dim]
};

}  // namespace

int main(int argc, char** argv) {
    if (argc != 3) {
        fprintf(stderr, "usage: llama_scalar MODEL.bin LOGITS.bin\n");
        return 2;
    }
    Reader in{fopen(argv[1], "rb")};
    if (!in.f) {
        perror(argv[1]);
        return 2;
    }
    const int layers = in.one<int32_t>(), hidden = in.one<int32_t>(), heads = in.one<int32_t>();
    const int kv_heads = in.one<int32_t>(), d = in.one<int32_t>(), inter = in.one<int32_t>();
    const int vocab = in.one<int32_t>(), tied = in.one<int32_t>(), scaled = in.one<int32_t>();
    const int original = in.one<int32_t>(), tokens = in.one<int32_t>();
    const double eps = in.one<double>(), theta = in.one<double>(), factor = in.one<double>();
    const double low = in.one<double>(), high = in.one<double>();
    std::vector<int32_t> ids(tokens);
    for (int t = 0; t < tokens; ++t) ids[t] = in.one<int32_t>();
    const std::vector<double> embedding = in.floats((size_t)vocab * hidden);
    std::vector<Layer> model(layers);
    for (Layer& l : model) {
        l.input_norm = in.floats(hidden);
        l.q = in.floats((size_t)heads * d * hidden);
        l.k = in.floats((size_t)kv_heads * d * hidden);
        l.v = in.floats((size_t)kv_heads * d * hidden);
        l.o = in.floats((size_t)hidden * heads * d);
        l.post_norm = in.floats(hidden);
        l.gate = in.floats((size_t)inter * hidden);
        l.up = in.floats((size_t)inter * hidden);
        l.down = in.floats((size_t)hidden * inter);
    }
    const std::vector<double> final_norm = in.floats(hidden);
    const std::vector<double> head = tied ? embedding : in.floats((size_t)vocab * hidden);
    fclose(in.f);

    // Inverse frequencies in 32-bit, Llama-3 scaled (src/cuda/dense_decoder.rs:1520-1544): a wavelength shorter than
    // original/high keeps its frequency, one longer than original/low is divided by the factor, between them the
    // two are blended.
    const int half = d / 2;
    std::vector<float> inv_freq(half);
    for (int i = 0; i < half; ++i) {
        const float exponent = (float)(2 * i) / (float)d;
        const float base = 1.0f / powf((float)theta, exponent);
        float freq = base;
        if (scaled) {
            const float wavelength = 6.283185307179586f / base;
            const float orig = (float)original, lo = (float)low, hi = (float)high, fac = (float)factor;
            if (wavelength < orig / hi) {
                freq = base;
            } else if (wavelength > orig / lo) {
                freq = base / fac;
            } else {
                const float smooth = (orig / wavelength - lo) / (hi - lo);
                freq = (1.0f - smooth) * base / fac + smooth * base;
            }
        }
        inv_freq[i] = freq;
    }

    const int group = heads / kv_heads;
    const double scale = 1.0 / std::sqrt((double)d);      // src/cuda/dense_decoder/flat_kv.rs:165
    FILE* out = fopen(argv[2], "wb");
    if (!out) {
        perror(argv[2]);
        return 2;
    }
    for (int t = 0; t < tokens; ++t) {
        // the token's row of the embedding table, no scale (src/cuda/kernels.rs:10-24)
        std::vector<double> residual(embedding.begin() + (size_t)ids[t] * hidden,
                                     embedding.begin() + (size_t)(ids[t] + 1) * hidden);
        // cos and sin of float(position) * frequency, the 32-bit table entries (src/cuda/dense_decoder.rs:1549-1556)
        std::vector<double> cosine(half), sine(half);
        for (int i = 0; i < half; ++i) {
            const float angle = (float)t * inv_freq[i];
            cosine[i] = (double)(float)std::cos((double)angle);
            sine[i] = (double)(float)std::sin((double)angle);
        }
        for (Layer& l : model) {
            const std::vector<double> x = rms_norm(residual, l.input_norm, eps);
            std::vector<double> q = times_transposed(l.q, x, heads * d, hidden);
            std::vector<double> k = times_transposed(l.k, x, kv_heads * d, hidden);
            const std::vector<double> v = times_transposed(l.v, x, kv_heads * d, hidden);
            // rotate-half on every head of q and k: (lo, hi) -> (lo cos - hi sin, hi cos + lo sin)
            // (src/cuda/kernels.rs:210-242, 244-282); the key is stored rotated (src/cuda/kernels.rs:283-337)
            for (int pass = 0; pass < 2; ++pass) {
                std::vector<double>& vec = pass == 0 ? q : k;
                const int count = pass == 0 ? heads : kv_heads;
                for (int h = 0; h < count; ++h)
                    for (int i = 0; i < half; ++i) {
                        const double lo = vec[h * d + i], hi = vec[h * d + half + i];
                        vec[h * d + i] = lo * cosine[i] - hi * sine[i];
                        vec[h * d + half + i] = hi * cosine[i] + lo * sine[i];
                    }
            }
            l.keys.push_back(k);
            l.values.push_back(v);
            // every query head over all keys so far, its own included (src/cuda/kernels.rs:447-562); query head h
            // reads kv head h / group
            std::vector<double> attended((size_t)heads * d, 0.0);
            for (int h = 0; h < heads; ++h) {
                const int kh = h / group;
                std::vector<double> score(t + 1);
                double top = -INFINITY;
                for (int j = 0; j <= t; ++j) {
                    double dot = 0.0;
                    for (int i = 0; i < d; ++i) dot += q[h * d + i] * l.keys[j][kh * d + i];
                    score[j] = dot * scale;
                    if (score[j] > top) top = score[j];
                }
                double total = 0.0;
                for (int j = 0; j <= t; ++j) {
                    score[j] = std::exp(score[j] - top);
                    total += score[j];
                }
                for (int j = 0; j <= t; ++j)
                    for (int i = 0; i < d; ++i) attended[h * d + i] += score[j] / total * l.values[j][kh * d + i];
            }
            const std::vector<double> projected = times_transposed(l.o, attended, hidden, heads * d);
            for (int i = 0; i < hidden; ++i) residual[i] += projected[i];
            const std::vector<double> m = rms_norm(residual, l.post_norm, eps);
            // down( silu(gate) * up )   (src/cuda/dense_decoder.rs:737-774, src/cuda/kernels.rs:191-208)
            const std::vector<double> g = times_transposed(l.gate, m, inter, hidden);
            const std::vector<double> u = times_transposed(l.up, m, inter, hidden);
            std::vector<double> activated(inter);
            for (int i = 0; i < inter; ++i) activated[i] = g[i] / (1.0 + std::exp(-g[i])) * u[i];
            const std::vector<double> fed = times_transposed(l.down, activated, hidden, inter);
            for (int i = 0; i < hidden; ++i) residual[i] += fed[i];
        }
        const std::vector<double> last = rms_norm(residual, final_norm, eps);
        const std::vector<double> logits = times_transposed(head, last, vocab, hidden);
        fwrite(logits.data(), sizeof(double), logits.size(), out);
    }
    fclose(out);
    return 0;
}
