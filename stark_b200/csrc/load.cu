// stark_b200_load: a converted-model directory (config.json + model.safetensors in the reference's own layout)
// straight into a dense decoder, for callers that are not Python.  The counterpart of the reference's
// `stark_glm_load(path_utf8, path_len, options, &model)` (vendor/glm-exl3-bridge/include/stark_glm.h:85-87) and of
// its artifact loader: config.json as `LanguageModelConfig` (crates/stark-engine/src/config/model/language_model.rs:5-11),
// model.safetensors through the bounded header reader (parameters/safetensors_metadata.rs:117-132, header <= 100 MB),
// per-matrix specs in `__metadata__` under `<name>.spec` (parameters/loader.rs:399-408), fused [q; k; v] and
// [up; gate] rows, planes either [rows, groups] or [groups, round_up4(rows)] (weight_matrix.rs:150-154), and the
// rule that every tensor of the file must be consumed (language_model/mod.rs:125).  Anything outside the dense
// decode path this engine implements is refused, never approximated.  Host code only: no kernel lives here.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "model.cuh"

namespace sb {

namespace {

// ---------------------------------------------------------------------------------------- a small JSON reader
struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0.0;
    bool integral = false;
    std::string str;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> fields;

    const Json *get(const char *name) const {
        if (kind != Object) return nullptr;
        for (auto &f : fields)
            if (f.first == name) return &f.second;
        return nullptr;
    }
    bool is_null() const { return kind == Null; }
};

struct JsonParser {
    const char *p, *end;
    int depth = 0;
    bool fail = false;

    void skip() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\r' || *p == '\t')) ++p;
    }
    bool literal(const char *word) {
        const size_t n = strlen(word);
        if ((size_t)(end - p) < n || memcmp(p, word, n) != 0) return false;
        p += n;
        return true;
    }
    bool string(std::string &out) {
        if (p >= end || *p != '"') return false;
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return false;
                switch (*p) {
                    case '"': out += '"'; break;
                    case '\\': out += '\\'; break;
                    case '/': out += '/'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'n': out += '\n'; break;
                    case 'r': out += '\r'; break;
                    case 't': out += '\t'; break;
                    case 'u': {
                        if (end - p < 5) return false;
                        unsigned code = 0;
                        for (int i = 1; i <= 4; ++i) {
                            const char c = p[i];
                            code <<= 4;
                            if (c >= '0' && c <= '9') code |= (unsigned)(c - '0');
                            else if (c >= 'a' && c <= 'f') code |= (unsigned)(c - 'a' + 10);
                            else if (c >= 'A' && c <= 'F') code |= (unsigned)(c - 'A' + 10);
                            else return false;
                        }
                        p += 4;
                        // names and enumerators of this format are ASCII; other code points are kept as UTF-8
                        if (code < 0x80) out += (char)code;
                        else if (code < 0x800) {
                            out += (char)(0xC0 | (code >> 6));
                            out += (char)(0x80 | (code & 0x3F));
                        } else {
                            out += (char)(0xE0 | (code >> 12));
                            out += (char)(0x80 | ((code >> 6) & 0x3F));
                            out += (char)(0x80 | (code & 0x3F));
                        }
                        break;
                    }
                    default: return false;
                }
                ++p;
            } else {
                out += *p++;
            }
        }
        if (p >= end) return false;
        ++p;
        return true;
    }
    Json value() {
        Json v;
        skip();
        if (p >= end || ++depth > 64) {
            fail = true;
            return v;
        }
        const char c = *p;
        if (c == '{') {
            v.kind = Json::Object;
            ++p;
            skip();
            if (p < end && *p == '}') {
                ++p;
            } else {
                for (;;) {
                    skip();
                    std::string key;
                    if (!string(key)) { fail = true; break; }
                    skip();
                    if (p >= end || *p != ':') { fail = true; break; }
                    ++p;
                    Json item = value();
                    if (fail) break;
                    for (auto &f : v.fields)
                        if (f.first == key) fail = true;  // a duplicate key is a malformed file
                    v.fields.emplace_back(std::move(key), std::move(item));
                    skip();
                    if (p < end && *p == ',') { ++p; continue; }
                    if (p < end && *p == '}') { ++p; break; }
                    fail = true;
                    break;
                }
            }
        } else if (c == '[') {
            v.kind = Json::Array;
            ++p;
            skip();
            if (p < end && *p == ']') {
                ++p;
            } else {
                for (;;) {
                    v.items.push_back(value());
                    if (fail) break;
                    skip();
                    if (p < end && *p == ',') { ++p; continue; }
                    if (p < end && *p == ']') { ++p; break; }
                    fail = true;
                    break;
                }
            }
        } else if (c == '"') {
            v.kind = Json::String;
            if (!string(v.str)) fail = true;
        } else if (c == 't') {
            v.kind = Json::Bool;
            v.b = true;
            if (!literal("true")) fail = true;
        } else if (c == 'f') {
            v.kind = Json::Bool;
            if (!literal("false")) fail = true;
        } else if (c == 'n') {
            if (!literal("null")) fail = true;
        } else {
            v.kind = Json::Number;
            const char *start = p;
            if (p < end && *p == '-') ++p;
            bool digits = false, frac = false;
            while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '+' || *p == '-')) {
                if (*p >= '0' && *p <= '9') digits = true;
                else frac = true;
                ++p;
            }
            if (!digits) {
                fail = true;
            } else {
                const std::string text(start, p);
                char *stop = nullptr;
                v.num = strtod(text.c_str(), &stop);
                v.integral = !frac;
                if (!stop || *stop) fail = true;
            }
        }
        --depth;
        return v;
    }
};

bool parse_json(const char *data, size_t size, Json &out) {
    JsonParser parser{data, data + size};
    out = parser.value();
    parser.skip();
    return !parser.fail && parser.p == parser.end;
}

bool read_file(const std::string &path, std::string &out, size_t limit) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return false;
    char buf[1 << 16];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) {
        out.append(buf, n);
        if (out.size() > limit) break;
    }
    const bool ok = !ferror(f) && out.size() <= limit;
    fclose(f);
    return ok;
}

struct Mapping {
    const uint8_t *data = nullptr;
    size_t size = 0;
    ~Mapping() {
        if (data) munmap(const_cast<uint8_t *>(data), size);
    }
    bool open_file(const std::string &path) {
        const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
        if (fd < 0) return false;
        struct stat st;
        if (fstat(fd, &st) != 0 || st.st_size <= 0) {
            ::close(fd);
            return false;
        }
        void *p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
        ::close(fd);
        if (p == MAP_FAILED) return false;
        data = static_cast<const uint8_t *>(p);
        size = (size_t)st.st_size;
        return true;
    }
};

// ---------------------------------------------------------------------------------------- config checks
bool is_str(const Json *v, const char *s) { return v && v->kind == Json::String && v->str == s; }
bool is_none(const Json *v) { return !v || v->is_null(); }
bool is_false(const Json *v) { return v && v->kind == Json::Bool && !v->b; }
bool is_true(const Json *v) { return v && v->kind == Json::Bool && v->b; }
bool as_u32(const Json *v, uint32_t &out) {
    if (!v || v->kind != Json::Number || !v->integral || v->num < 0 || v->num > 4294967295.0) return false;
    out = (uint32_t)v->num;
    return true;
}

bool same(const Json &a, const Json &b) {
    if (a.kind != b.kind) return false;
    switch (a.kind) {
        case Json::Null: return true;
        case Json::Bool: return a.b == b.b;
        case Json::Number: return a.num == b.num;
        case Json::String: return a.str == b.str;
        case Json::Array:
            if (a.items.size() != b.items.size()) return false;
            for (size_t i = 0; i < a.items.size(); ++i)
                if (!same(a.items[i], b.items[i])) return false;
            return true;
        case Json::Object:
            if (a.fields.size() != b.fields.size()) return false;
            for (auto &f : a.fields) {
                const Json *o = b.get(f.first.c_str());
                if (!o || !same(f.second, *o)) return false;
            }
            return true;
    }
    return false;
}

// The norm form the dense path implements: scale only, no offset, no mean subtraction (read_artifact's checks).
bool plain_norm(const Json *n, const Json &reference) {
    return n && same(*n, reference) && is_none(n->get("scale_offset")) && is_false(n->get("subtract_mean")) &&
           is_true(n->get("has_scale")) && is_false(n->get("has_biases"));
}

struct Tensor {
    std::string dtype;
    std::vector<uint64_t> shape;
    uint64_t lo = 0, hi = 0;
};

struct Artifact {
    stark_b200_dense_config cfg{};
    uint32_t max_sequence = 32768;
    Mapping file;
    const uint8_t *payload = nullptr;
    size_t payload_size = 0;
    std::map<std::string, Tensor> tensors;
    std::map<std::string, std::string> metadata;
    std::set<std::string> used;
};

stark_b200_status read_config(const std::string &dir, Artifact &a) {
    std::string text;
    if (!read_file(dir + "/config.json", text, 64u << 20)) return STARK_B200_IO_FAILURE;
    Json root;
    if (!parse_json(text.data(), text.size(), root)) return STARK_B200_INVALID_ARGUMENT;
    if (!is_str(root.get("type"), "LanguageModelConfig")) return STARK_B200_UNSUPPORTED;
    const Json *dec = root.get("decoder_config");
    const Json *tr = dec ? dec->get("transformer_config") : nullptr;
    const Json *layers = tr ? tr->get("layer_configs") : nullptr;
    const Json *emb = dec ? dec->get("embedding_config") : nullptr;
    if (!layers || layers->kind != Json::Array || layers->items.empty() || !emb) return STARK_B200_UNSUPPORTED;
    const Json &first = layers->items[0];
    const Json *mixer = first.get("mixer_config"), *rope = first.get("rope_config"), *norm = first.get("pre_mixer_norm_config");
    if (!mixer || !rope || !norm) return STARK_B200_UNSUPPORTED;
    if (is_str(emb->get("type"), "TiedEmbeddingConfig")) a.cfg.tied = 1;
    else if (is_str(emb->get("type"), "UntiedEmbeddingConfig")) a.cfg.tied = 0;
    else return STARK_B200_UNSUPPORTED;
    for (const char *key : {"input_scale", "logit_soft_cap", "logit_scale"})
        if (!is_none(emb->get(key))) return STARK_B200_UNSUPPORTED;
    if (!is_none(dec->get("ple_model_config")) || !is_none(dec->get("embedding_norm_config"))) return STARK_B200_UNSUPPORTED;
    for (const Json &lc : layers->items) {
        if (!same(lc, first)) return STARK_B200_UNSUPPORTED;  // layers that differ from one another
        const Json *m = lc.get("mixer_config");
        if (!m || !is_str(m->get("type"), "AttentionConfig") || !is_true(m->get("is_causal")) || !is_none(m->get("scale")))
            return STARK_B200_UNSUPPORTED;
        if (!is_none(m->get("sliding_window_size")) || !is_none(m->get("logit_soft_cap")) || !is_false(m->get("has_sinks")))
            return STARK_B200_UNSUPPORTED;
        for (const char *key : {"has_qkvg_biases", "has_out_biases", "has_gate", "normalize_values", "is_kv_sharing"})
            if (!is_false(m->get(key))) return STARK_B200_UNSUPPORTED;
        const Json *mlp = lc.get("mlp_config");
        const Json *act = mlp ? mlp->get("activation") : nullptr;
        if (!mlp || !is_str(mlp->get("type"), "DenseMLPConfig") || !act || !is_str(act->get("type"), "SiLU"))
            return STARK_B200_UNSUPPORTED;
        const Json *rc = lc.get("rope_config");
        if (!rc || !is_str(rc->get("type"), "UnscaledRoPEConfig")) return STARK_B200_UNSUPPORTED;
        for (const char *key : {"mixer_conv_config", "post_mixer_norm_config", "mlp_conv_config", "post_mlp_norm_config",
                                "ple_config", "kv_source_layer_index"})
            if (!is_none(lc.get(key))) return STARK_B200_UNSUPPORTED;
        for (const Json *n : {lc.get("pre_mixer_norm_config"), lc.get("pre_mlp_norm_config"), m->get("query_norm_config"),
                              m->get("key_norm_config")})
            if (!plain_norm(n, *norm)) return STARK_B200_UNSUPPORTED;
    }
    const Json *out_norm = tr->get("output_norm_config");
    if (!out_norm || !same(*out_norm, *norm)) return STARK_B200_UNSUPPORTED;
    a.cfg.layers = (uint32_t)layers->items.size();
    const Json *eps = norm->get("epsilon"), *base = rope->get("base");
    if (!as_u32(tr->get("model_dim"), a.cfg.hidden) || !as_u32(mixer->get("num_heads"), a.cfg.q_heads) ||
        !as_u32(mixer->get("num_groups"), a.cfg.kv_heads) || !as_u32(mixer->get("head_dim"), a.cfg.head_dim) ||
        !as_u32(tr->get("hidden_dim"), a.cfg.inter) || !as_u32(dec->get("vocab_size"), a.cfg.vocab) || !eps ||
        eps->kind != Json::Number || !base || base->kind != Json::Number)
        return STARK_B200_INVALID_ARGUMENT;
    a.cfg.eps = (float)eps->num;
    a.cfg.rope_theta = (float)base->num;
    if (a.cfg.head_dim != kHeadDim) return STARK_B200_UNSUPPORTED;
    uint32_t seq = 0;
    if (as_u32(rope->get("max_sequence_length"), seq) && seq) a.max_sequence = seq;
    return STARK_B200_OK;
}

stark_b200_status read_safetensors(const std::string &path, Artifact &a) {
    if (!a.file.open_file(path)) return STARK_B200_IO_FAILURE;
    if (a.file.size < 8) return STARK_B200_INVALID_ARGUMENT;
    uint64_t n = 0;
    memcpy(&n, a.file.data, 8);
    if (n > 100ull * 1024 * 1024 || 8 + n > a.file.size) return STARK_B200_INVALID_ARGUMENT;  // safetensors_metadata.rs:117-132
    Json header;
    if (!parse_json(reinterpret_cast<const char *>(a.file.data + 8), (size_t)n, header) || header.kind != Json::Object)
        return STARK_B200_INVALID_ARGUMENT;
    a.payload = a.file.data + 8 + n;
    a.payload_size = a.file.size - 8 - (size_t)n;
    for (auto &f : header.fields) {
        if (f.first == "__metadata__") {
            if (f.second.kind == Json::Object)
                for (auto &mf : f.second.fields)
                    if (mf.second.kind == Json::String) a.metadata[mf.first] = mf.second.str;
            continue;
        }
        Tensor t;
        const Json *dtype = f.second.get("dtype"), *shape = f.second.get("shape"), *offs = f.second.get("data_offsets");
        if (!dtype || dtype->kind != Json::String || !shape || shape->kind != Json::Array || !offs ||
            offs->kind != Json::Array || offs->items.size() != 2)
            return STARK_B200_INVALID_ARGUMENT;
        t.dtype = dtype->str;
        for (auto &d : shape->items) {
            if (d.kind != Json::Number || !d.integral || d.num < 0) return STARK_B200_INVALID_ARGUMENT;
            t.shape.push_back((uint64_t)d.num);
        }
        if (offs->items[0].kind != Json::Number || offs->items[1].kind != Json::Number || offs->items[0].num < 0 ||
            offs->items[1].num < offs->items[0].num)
            return STARK_B200_INVALID_ARGUMENT;
        t.lo = (uint64_t)offs->items[0].num;
        t.hi = (uint64_t)offs->items[1].num;
        a.tensors[f.first] = std::move(t);
    }
    return STARK_B200_OK;
}

// The bytes of tensor `name`, which must have exactly this dtype and shape and consistent offsets.
const uint8_t *tensor_bytes(Artifact &a, const std::string &name, const char *dtype, std::vector<uint64_t> shape,
                            uint32_t element_bytes) {
    auto it = a.tensors.find(name);
    if (it == a.tensors.end() || it->second.dtype != dtype || it->second.shape != shape) return nullptr;
    uint64_t bytes = element_bytes;
    for (uint64_t d : shape) bytes *= d;
    if (it->second.hi - it->second.lo != bytes || it->second.hi > a.payload_size) return nullptr;
    a.used.insert(name);
    return a.payload + it->second.lo;
}

stark_b200_status load_matrix(Artifact &a, stark_b200_model *model, uint32_t layer, uint32_t which, const std::string &name,
                              uint32_t rows, uint32_t columns) {
    auto spec_text = a.metadata.find(name + ".spec");
    Json spec;
    if (spec_text == a.metadata.end() || !parse_json(spec_text->second.data(), spec_text->second.size(), spec))
        return STARK_B200_UNSUPPORTED;
    uint32_t group = 0, bits = 0;
    if (!is_str(spec.get("type"), "MLXSpec") || !as_u32(spec.get("group_size"), group) || group != 64 ||
        !as_u32(spec.get("bits"), bits) || bits != 4)
        return STARK_B200_UNSUPPORTED;  // the decoder's matvec kernels are written for 4-bit group-64 matrices
    const uint32_t groups = columns / 64u;
    stark_b200_affine_desc d{};
    d.struct_size = sizeof(d);
    d.abi_version = STARK_B200_ABI_VERSION;
    d.rows = rows;
    d.columns = columns;
    d.bits = bits;
    d.group = 64;
    d.plane_kind = STARK_B200_PLANE_BF16;
    d.location = STARK_B200_HOST;
    std::vector<uint64_t> plane_shape;
    const Json *layout = spec.get("layout");
    if (is_str(layout, "input_output")) {
        plane_shape = {rows, groups};
    } else if (is_str(layout, "output_input")) {
        d.scale_layout = 1;
        d.plane_pitch = rows + ((4u - rows % 4u) % 4u);
        plane_shape = {groups, d.plane_pitch};
    } else {
        return STARK_B200_UNSUPPORTED;
    }
    const uint8_t *codes = tensor_bytes(a, name + ".weights", "U8", {rows, (uint64_t)columns * bits / 8u}, 1);
    const uint8_t *scales = tensor_bytes(a, name + ".scales", "BF16", plane_shape, 2);
    const uint8_t *biases = tensor_bytes(a, name + ".biases", "BF16", plane_shape, 2);
    if (!codes || !scales || !biases) return STARK_B200_INVALID_ARGUMENT;
    if (!model) return STARK_B200_OK;  // validation pass
    return stark_b200_model_set_affine(model, layer, which, codes, scales, biases, &d);
}

stark_b200_status load_vector(Artifact &a, stark_b200_model *model, uint32_t layer, uint32_t which, const std::string &name,
                              uint32_t width) {
    const uint8_t *data = tensor_bytes(a, name + ".scales", "F32", {width}, 4);
    if (!data) return STARK_B200_INVALID_ARGUMENT;
    if (!model) return STARK_B200_OK;  // validation pass
    return stark_b200_model_set_vector(model, layer, which, reinterpret_cast<const float *>(data), width);
}

}  // namespace

}  // namespace sb

using namespace sb;

extern "C" stark_b200_status stark_b200_load(const uint8_t *path_utf8, size_t path_len, const stark_b200_load_options *options,
                                             stark_b200_model **out_model) {
    if (!path_utf8 || !path_len || !options || !out_model) return STARK_B200_INVALID_ARGUMENT;
    if (options->struct_size != sizeof(stark_b200_load_options) || options->abi_version != STARK_B200_ABI_VERSION)
        return STARK_B200_ABI_MISMATCH;
    *out_model = nullptr;
    const std::string dir(reinterpret_cast<const char *>(path_utf8), path_len);
    auto artifact = std::make_unique<Artifact>();
    Artifact &a = *artifact;
    stark_b200_status st = read_config(dir, a);
    if (st != STARK_B200_OK) return st;
    if ((st = read_safetensors(dir + "/model.safetensors", a)) != STARK_B200_OK) return st;
    uint64_t context = options->context_tokens ? options->context_tokens : a.max_sequence;
    if (context > a.max_sequence) return STARK_B200_CONTEXT_LIMIT;
    a.cfg.struct_size = sizeof(a.cfg);
    a.cfg.abi_version = STARK_B200_ABI_VERSION;
    a.cfg.context_tokens = (uint32_t)context;
    const auto &c = a.cfg;
    const uint32_t qw = c.q_heads * c.head_dim, kw = c.kv_heads * c.head_dim;
    // Every tensor the decoder reads, in one place: walked once without a model (names, specs, types, shapes and
    // offsets are checked and the all-consumed rule applied before any device memory is touched), then again to
    // upload.
    auto walk = [&](stark_b200_model *model) -> stark_b200_status {
        stark_b200_status s;
        if (c.tied) {
            if ((s = load_matrix(a, model, 0, STARK_B200_MAT_EMBED, "decoder.embedding.embedding", c.vocab, c.hidden)) != STARK_B200_OK) return s;
        } else {
            if ((s = load_matrix(a, model, 0, STARK_B200_MAT_EMBED, "decoder.embedding.input_embedding", c.vocab, c.hidden)) != STARK_B200_OK) return s;
            if ((s = load_matrix(a, model, 0, STARK_B200_MAT_LM_HEAD, "decoder.embedding.output_embedding", c.vocab, c.hidden)) != STARK_B200_OK) return s;
        }
        for (uint32_t i = 0; i < c.layers; ++i) {
            const std::string p = "decoder.transformer.layers." + std::to_string(i);
            if ((s = load_vector(a, model, i, STARK_B200_VEC_ATTN_NORM, p + ".pre_mixer_norm", c.hidden)) != STARK_B200_OK) return s;
            if ((s = load_vector(a, model, i, STARK_B200_VEC_MLP_NORM, p + ".pre_mlp_norm", c.hidden)) != STARK_B200_OK) return s;
            if ((s = load_vector(a, model, i, STARK_B200_VEC_Q_NORM, p + ".mixer.query_norm", c.head_dim)) != STARK_B200_OK) return s;
            if ((s = load_vector(a, model, i, STARK_B200_VEC_K_NORM, p + ".mixer.key_norm", c.head_dim)) != STARK_B200_OK) return s;
            if ((s = load_matrix(a, model, i, STARK_B200_MAT_QKV, p + ".mixer.qkvg_projection.weights", qw + 2u * kw, c.hidden)) != STARK_B200_OK) return s;
            if ((s = load_matrix(a, model, i, STARK_B200_MAT_O, p + ".mixer.out_projection.weights", c.hidden, qw)) != STARK_B200_OK) return s;
            if ((s = load_matrix(a, model, i, STARK_B200_MAT_UPGATE, p + ".mlp.up_projection.weights", 2u * c.inter, c.hidden)) != STARK_B200_OK) return s;
            if ((s = load_matrix(a, model, i, STARK_B200_MAT_DOWN, p + ".mlp.down_projection.weights", c.hidden, c.inter)) != STARK_B200_OK) return s;
        }
        return load_vector(a, model, 0, STARK_B200_VEC_FINAL_NORM, "decoder.transformer.output_norm", c.hidden);
    };
    if ((st = walk(nullptr)) != STARK_B200_OK) return st;
    if (a.used.size() != a.tensors.size()) return STARK_B200_INVALID_ARGUMENT;  // every tensor must be consumed
    stark_b200_model *model = nullptr;
    if ((st = stark_b200_model_create(&a.cfg, &model)) != STARK_B200_OK) return st;
    auto fail = [&](stark_b200_status s) {
        stark_b200_destroy(&model);
        return s;
    };
    if ((st = walk(model)) != STARK_B200_OK) return fail(st);
    if ((st = stark_b200_model_finalize(model)) != STARK_B200_OK) return fail(st);
    *out_model = model;
    return STARK_B200_OK;
}
