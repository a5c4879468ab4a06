// C-ABI: tq_model_load over a converted TurboQuant model directory.
//
// A shard is a safetensors file: 8-byte little-endian header length, a JSON header
// {name: {dtype, shape, data_offsets}, "__metadata__": {...}}, then the tensor bytes.  Shards whose
// metadata says quantization_method = "turboquant" hold, per quantised weight, {name}.packed_primary,
// .packed_residual, .norms, .seeds, model-level tq_codebook_primary / tq_codebook_residual and, when
// tq_per_layer_codebooks = "true", {name}.codebook_primary / .codebook_residual
// (src/serialization.cpp:19-97).  Loading rules follow src/turboquant_c_dequant.cpp:68-150: companion
// *_passthrough shards and shards without the marker are skipped, the WHT block is seeds[2] (512 when
// absent), per-layer codebooks win only when the metadata announces them.  Every layer becomes a
// device-resident linear handle (tq_linear_create); only the tensors needed are read from disk.
#include <dirent.h>
#include <sys/stat.h>

#include <algorithm>
#include <cctype>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "tq_host.hpp"
#include "turboquant_c/turboquant_b200.h"
#include "turboquant_c/turboquant_c.h"

namespace {

using tq::Error;

// ---- a JSON reader sufficient for safetensors headers ----
struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    double number = 0;
    bool boolean = false;
    std::string text;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;

    const Json* find(const std::string& key) const {
        for (const auto& m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
};

class JsonReader {
public:
    JsonReader(const char* p, size_t n) : p_(p), end_(p + n) {}
    Json parse() {
        Json v = value(0);
        skip();
        if (p_ != end_) throw Error("safetensors header: trailing characters");
        return v;
    }

private:
    void skip() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
    }
    char peek() {
        skip();
        if (p_ >= end_) throw Error("safetensors header: unexpected end");
        return *p_;
    }
    void expect(char c) {
        if (peek() != c) throw Error(std::string("safetensors header: expected '") + c + "'");
        ++p_;
    }
    std::string string() {
        expect('"');
        std::string out;
        while (true) {
            if (p_ >= end_) throw Error("safetensors header: unterminated string");
            const char c = *p_++;
            if (c == '"') return out;
            if (c != '\\') {
                out.push_back(c);
                continue;
            }
            if (p_ >= end_) throw Error("safetensors header: bad escape");
            const char e = *p_++;
            switch (e) {
                case '"': out.push_back('"'); break;
                case '\\': out.push_back('\\'); break;
                case '/': out.push_back('/'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'n': out.push_back('\n'); break;
                case 'r': out.push_back('\r'); break;
                case 't': out.push_back('\t'); break;
                case 'u': {
                    if (end_ - p_ < 4) throw Error("safetensors header: bad \\u escape");
                    const unsigned cp = static_cast<unsigned>(std::strtoul(std::string(p_, p_ + 4).c_str(), nullptr, 16));
                    p_ += 4;
                    // tensor names are ASCII in practice; other code points are kept as UTF-8 (no surrogate pairing)
                    if (cp < 0x80) out.push_back(static_cast<char>(cp));
                    else if (cp < 0x800) {
                        out.push_back(static_cast<char>(0xC0 | (cp >> 6)));
                        out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
                    } else {
                        out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
                        out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
                        out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
                    }
                    break;
                }
                default: throw Error("safetensors header: bad escape");
            }
        }
    }
    Json value(int depth) {
        if (depth > 16) throw Error("safetensors header: nesting too deep");
        Json v;
        const char c = peek();
        if (c == '{') {
            ++p_;
            v.kind = Json::Object;
            if (peek() == '}') {
                ++p_;
                return v;
            }
            while (true) {
                std::string key = string();
                expect(':');
                v.members.emplace_back(std::move(key), value(depth + 1));
                if (peek() == ',') {
                    ++p_;
                    continue;
                }
                expect('}');
                return v;
            }
        }
        if (c == '[') {
            ++p_;
            v.kind = Json::Array;
            if (peek() == ']') {
                ++p_;
                return v;
            }
            while (true) {
                v.items.push_back(value(depth + 1));
                if (peek() == ',') {
                    ++p_;
                    continue;
                }
                expect(']');
                return v;
            }
        }
        if (c == '"') {
            v.kind = Json::String;
            v.text = string();
            return v;
        }
        auto literal = [&](const char* word) {
            const size_t n = std::char_traits<char>::length(word);
            if (static_cast<size_t>(end_ - p_) < n || std::string(p_, p_ + n) != word) throw Error("safetensors header: bad literal");
            p_ += n;
        };
        if (c == 't') { literal("true"); v.kind = Json::Bool; v.boolean = true; return v; }
        if (c == 'f') { literal("false"); v.kind = Json::Bool; return v; }
        if (c == 'n') { literal("null"); return v; }
        const char* start = p_;
        while (p_ < end_ && (std::isdigit(static_cast<unsigned char>(*p_)) || *p_ == '-' || *p_ == '+' || *p_ == '.' || *p_ == 'e' || *p_ == 'E')) ++p_;
        if (p_ == start) throw Error("safetensors header: unexpected character");
        v.kind = Json::Number;
        v.number = std::strtod(std::string(start, p_).c_str(), nullptr);
        return v;
    }
    const char* p_;
    const char* end_;
};

struct TensorInfo {
    std::string dtype;
    std::vector<long> shape;
    unsigned long long begin = 0, end = 0;
    size_t count() const {
        size_t n = 1;
        for (long d : shape) n *= static_cast<size_t>(d);
        return n;
    }
};

struct FileCloser {
    void operator()(std::FILE* f) const {
        if (f) std::fclose(f);
    }
};

struct Shard {
    std::unique_ptr<std::FILE, FileCloser> file;
    unsigned long long data_start = 0, data_bytes = 0;
    std::map<std::string, TensorInfo> tensors;
    std::map<std::string, std::string> metadata;

    explicit Shard(const std::string& path) : file(std::fopen(path.c_str(), "rb")) {
        if (!file) throw Error("cannot open " + path);
        unsigned char len[8];
        if (std::fread(len, 1, 8, file.get()) != 8) throw Error(path + ": not a safetensors file");
        unsigned long long n = 0;
        for (int i = 7; i >= 0; --i) n = (n << 8) | len[i];
        struct stat sb;
        if (stat(path.c_str(), &sb) != 0 || n > static_cast<unsigned long long>(sb.st_size) - 8 || n > (100ull << 20))
            throw Error(path + ": header length out of range");
        std::string header(static_cast<size_t>(n), '\0');
        if (std::fread(&header[0], 1, header.size(), file.get()) != header.size()) throw Error(path + ": truncated header");
        data_start = 8 + n;
        data_bytes = static_cast<unsigned long long>(sb.st_size) - data_start;
        const Json root = JsonReader(header.data(), header.size()).parse();
        if (root.kind != Json::Object) throw Error(path + ": header is not an object");
        for (const auto& m : root.members) {
            if (m.first == "__metadata__") {
                if (m.second.kind == Json::Object)
                    for (const auto& kv : m.second.members)
                        if (kv.second.kind == Json::String) metadata[kv.first] = kv.second.text;
                continue;
            }
            const Json *dt = m.second.find("dtype"), *sh = m.second.find("shape"), *off = m.second.find("data_offsets");
            if (!dt || dt->kind != Json::String || !sh || sh->kind != Json::Array || !off || off->kind != Json::Array ||
                off->items.size() != 2)
                throw Error(path + ": malformed entry for tensor " + m.first);
            TensorInfo t;
            t.dtype = dt->text;
            for (const Json& d : sh->items) {
                if (d.kind != Json::Number || d.number < 0) throw Error(path + ": bad shape for tensor " + m.first);
                t.shape.push_back(static_cast<long>(d.number));
            }
            t.begin = static_cast<unsigned long long>(off->items[0].number);
            t.end = static_cast<unsigned long long>(off->items[1].number);
            if (t.begin > t.end || t.end > data_bytes) throw Error(path + ": tensor " + m.first + " points outside the file");
            tensors[m.first] = std::move(t);
        }
    }

    // The bytes of tensor `name`, checked against the expected dtype and element size.
    std::vector<unsigned char> read(const std::string& name, const char* dtype, size_t elem_bytes) const {
        const auto it = tensors.find(name);
        if (it == tensors.end()) throw Error("missing tensor " + name);
        const TensorInfo& t = it->second;
        if (t.dtype != dtype) throw Error("tensor " + name + " has dtype " + t.dtype + ", expected " + dtype);
        if (t.end - t.begin != t.count() * elem_bytes) throw Error("tensor " + name + ": byte size does not match its shape");
        std::vector<unsigned char> out(static_cast<size_t>(t.end - t.begin));
        if (fseeko(file.get(), static_cast<off_t>(data_start + t.begin), SEEK_SET) != 0 ||
            (!out.empty() && std::fread(out.data(), 1, out.size(), file.get()) != out.size()))
            throw Error("tensor " + name + ": short read");
        return out;
    }
};

bool ends_with(const std::string& s, const std::string& suffix) {
    return s.size() >= suffix.size() && s.compare(s.size() - suffix.size(), suffix.size(), suffix) == 0;
}

}  // namespace

struct tq_model_s {
    std::string path;
    std::vector<std::string> names;
    std::vector<tq_linear_t> layers;
    ~tq_model_s() {
        for (tq_linear_t l : layers) tq_linear_free(l);
    }
};

namespace {

void load_shard(const std::string& path, tq_model_s& model) {
    const Shard shard(path);
    const auto method = shard.metadata.find("quantization_method");
    if (method == shard.metadata.end() || method->second != "turboquant") return;
    const std::vector<unsigned char> shared_p = shard.read("tq_codebook_primary", "F32", 4);
    const std::vector<unsigned char> shared_r = shard.read("tq_codebook_residual", "F32", 4);
    const auto flag = shard.metadata.find("tq_per_layer_codebooks");
    const bool per_layer = flag != shard.metadata.end() && flag->second == "true";
    const std::string suffix = ".packed_primary";
    for (const auto& entry : shard.tensors) {
        if (!ends_with(entry.first, suffix)) continue;
        const std::string layer = entry.first.substr(0, entry.first.size() - suffix.size());
        const TensorInfo& pp_info = entry.second;
        const auto pr_it = shard.tensors.find(layer + ".packed_residual");
        if (pr_it == shard.tensors.end()) throw Error(path + ": " + layer + " lacks .packed_residual");
        const TensorInfo& pr_info = pr_it->second;
        if (pp_info.shape.size() != 2 || pr_info.shape.size() != 2 || pp_info.shape[0] != pr_info.shape[0] ||
            (pp_info.shape[1] != pr_info.shape[1] && pp_info.shape[1] != 2 * pr_info.shape[1]))
            throw Error(path + ": " + layer + " has inconsistent plane shapes");
        const long out = pp_info.shape[0], in = pr_info.shape[1] * 2;
        if (out <= 0 || in <= 0 || out > (1l << 30) || in > (1l << 30)) throw Error(path + ": " + layer + " has unusable dimensions");
        const std::vector<unsigned char> pp = shard.read(layer + ".packed_primary", "U8", 1);
        const std::vector<unsigned char> pr = shard.read(layer + ".packed_residual", "U8", 1);
        const std::vector<unsigned char> norms = shard.read(layer + ".norms", "F32", 4);
        const std::vector<unsigned char> seeds_raw = shard.read(layer + ".seeds", "U32", 4);
        if (norms.size() != static_cast<size_t>(out) * 4) throw Error(path + ": " + layer + ".norms does not have one entry per row");
        uint32_t seeds[3] = {0, 0, 512};   // block size 512 when the tensor is short (src/turboquant_c_dequant.cpp:124)
        for (size_t i = 0; i < 3 && (i + 1) * 4 <= seeds_raw.size(); ++i) std::memcpy(&seeds[i], seeds_raw.data() + 4 * i, 4);
        std::vector<unsigned char> cp = shared_p, cr = shared_r;
        if (per_layer) {
            if (shard.tensors.count(layer + ".codebook_primary")) cp = shard.read(layer + ".codebook_primary", "F32", 4);
            if (shard.tensors.count(layer + ".codebook_residual")) cr = shard.read(layer + ".codebook_residual", "F32", 4);
        }
        tq_linear_t lin = tq_linear_create(static_cast<int>(in), static_cast<int>(out), pp.data(), static_cast<int>(pp_info.shape[1]),
                                           pr.data(), reinterpret_cast<const float*>(norms.data()), seeds,
                                           reinterpret_cast<const float*>(cp.data()), static_cast<int>(cp.size() / 4),
                                           reinterpret_cast<const float*>(cr.data()), static_cast<int>(cr.size() / 4), seeds[2]);
        if (!lin) throw Error(path + ": " + layer + ": " + tq_last_error());
        model.names.push_back(layer);
        model.layers.push_back(lin);
    }
}


// ---- writing a dequantised model directory (src/turboquant_c_dequant.cpp:20-191) ----------------

void make_dirs(const std::string& path) {
    std::string cur;
    for (size_t i = 0; i <= path.size(); ++i) {
        if (i == path.size() || path[i] == '/') {
            if (!cur.empty() && cur != "/") {
                if (mkdir(cur.c_str(), 0777) != 0 && errno != EEXIST) throw Error("cannot create directory " + cur);
            }
        }
        if (i < path.size()) cur.push_back(path[i]);
    }
}

std::string read_file(const std::string& path) {
    std::unique_ptr<std::FILE, FileCloser> f(std::fopen(path.c_str(), "rb"));
    if (!f) throw Error("cannot open " + path);
    std::string out;
    char buf[1 << 16];
    size_t n;
    while ((n = std::fread(buf, 1, sizeof buf, f.get())) > 0) out.append(buf, n);
    return out;
}

void write_file(const std::string& path, const std::string& bytes) {
    std::unique_ptr<std::FILE, FileCloser> f(std::fopen(path.c_str(), "wb"));
    if (!f || (!bytes.empty() && std::fwrite(bytes.data(), 1, bytes.size(), f.get()) != bytes.size()))
        throw Error("cannot write " + path);
}

// The copied config.json loses its "quantization_config" object (with the comma before it), so
// that downstream loaders take the output for an ordinary model (:36-66).
std::string strip_quantization_config(std::string json) {
    const size_t qc = json.find("\"quantization_config\"");
    if (qc == std::string::npos) return json;
    const size_t open = json.find('{', qc);
    if (open == std::string::npos) return json;
    int depth = 1;
    size_t pos = open + 1;
    while (pos < json.size() && depth > 0) {
        if (json[pos] == '{') ++depth;
        else if (json[pos] == '}') --depth;
        ++pos;
    }
    const size_t comma = json.rfind(',', qc);
    if (comma != std::string::npos && comma < qc) json.erase(comma, pos - comma);
    return json;
}

struct OutTensor {
    std::string dtype;
    std::vector<long> shape;
    std::vector<unsigned char> bytes;
};

// A safetensors file: 8-byte little-endian header length, JSON header (padded with spaces to a
// multiple of 8), tensor bytes in name order.
void write_safetensors_file(const std::string& path, const std::map<std::string, OutTensor>& tensors) {
    std::string header = "{\"__metadata__\":{\"format\":\"mlx\"}";
    unsigned long long off = 0;
    for (const auto& kv : tensors) {
        header += ",\"";
        for (char c : kv.first) {
            if (c == '"' || c == '\\') header.push_back('\\');
            header.push_back(c);
        }
        header += "\":{\"dtype\":\"" + kv.second.dtype + "\",\"shape\":[";
        for (size_t i = 0; i < kv.second.shape.size(); ++i) header += (i ? "," : "") + std::to_string(kv.second.shape[i]);
        header += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + kv.second.bytes.size()) + "]}";
        off += kv.second.bytes.size();
    }
    header += "}";
    while (header.size() % 8) header.push_back(' ');
    std::unique_ptr<std::FILE, FileCloser> f(std::fopen(path.c_str(), "wb"));
    if (!f) throw Error("cannot write " + path);
    unsigned char len[8];
    unsigned long long n = header.size();
    for (int i = 0; i < 8; ++i) len[i] = static_cast<unsigned char>((n >> (8 * i)) & 0xff);
    bool ok = std::fwrite(len, 1, 8, f.get()) == 8 && std::fwrite(header.data(), 1, header.size(), f.get()) == header.size();
    for (const auto& kv : tensors)
        ok = ok && (kv.second.bytes.empty() || std::fwrite(kv.second.bytes.data(), 1, kv.second.bytes.size(), f.get()) == kv.second.bytes.size());
    if (!ok) throw Error("short write to " + path);
}

// fp32 -> bf16, round to nearest even (what a framework's astype does); NaN stays NaN.
uint16_t f32_to_bf16(uint32_t u) {
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x0040u);
    return static_cast<uint16_t>((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

void dequant_shard(const std::string& in_dir, const std::string& fname, const std::string& out_dir) {
    const std::string path = in_dir + "/" + fname;
    const Shard shard(path);
    const auto method = shard.metadata.find("quantization_method");
    if (method == shard.metadata.end() || method->second != "turboquant") {   // not ours: copied as it is (:77-82)
        write_file(out_dir + "/" + fname, read_file(path));
        return;
    }
    // The output dtype is the passthrough tensors' (they keep the source model's), bfloat16 without
    // a passthrough file (:152-163); the first tensor in name order decides.
    const std::string stem = fname.substr(0, fname.size() - std::string(".safetensors").size());
    const std::string pt_path = in_dir + "/" + stem + "_passthrough.safetensors";
    struct stat sb;
    std::unique_ptr<Shard> pt;
    if (stat(pt_path.c_str(), &sb) == 0) pt.reset(new Shard(pt_path));
    std::string target = "BF16";
    if (pt && !pt->tensors.empty()) target = pt->tensors.begin()->second.dtype;
    if (target != "BF16" && target != "F16" && target != "F32") target = "BF16";

    // every quantised layer of the shard becomes a device-resident linear (the loader's rules)
    tq_model_s model;
    load_shard(path, model);
    std::map<std::string, OutTensor> out;
    for (size_t i = 0; i < model.layers.size(); ++i) {
        tq_linear_t lin = model.layers[i];
        const long rows = tq_linear_out_features(lin), cols = tq_linear_in_features(lin);
        OutTensor t;
        t.dtype = target;
        t.shape = {rows, cols};
        const size_t n = static_cast<size_t>(rows) * cols;
        if (target == "F16") {
            t.bytes.resize(n * 2);
            if (tq_linear_dequantize(lin, t.bytes.data(), TQ_F16, nullptr) != 0) throw Error(model.names[i] + ": " + tq_last_error());
        } else {
            std::vector<uint32_t> w(n);
            if (tq_linear_dequantize(lin, w.data(), TQ_F32, nullptr) != 0) throw Error(model.names[i] + ": " + tq_last_error());
            if (target == "F32") {
                t.bytes.resize(n * 4);
                std::memcpy(t.bytes.data(), w.data(), n * 4);
            } else {
                t.bytes.resize(n * 2);
                uint16_t* o = reinterpret_cast<uint16_t*>(t.bytes.data());
                for (size_t k = 0; k < n; ++k) o[k] = f32_to_bf16(w[k]);
            }
        }
        out[model.names[i] + ".weight"] = std::move(t);
    }
    // passthrough tensors (layers kept unquantised) are merged under their own names (:172-179)
    if (pt) {
        for (const auto& kv : pt->tensors) {
            if (out.count(kv.first)) continue;
            OutTensor t;
            t.dtype = kv.second.dtype;
            t.shape = kv.second.shape;
            const size_t es = kv.second.count() ? static_cast<size_t>(kv.second.end - kv.second.begin) / kv.second.count() : 1;
            t.bytes = pt->read(kv.first, kv.second.dtype.c_str(), es);
            out[kv.first] = std::move(t);
        }
    }
    write_safetensors_file(out_dir + "/" + fname, out);
}

void dequant_model_dir(const std::string& in_dir, const std::string& out_dir) {
    make_dirs(out_dir);
    std::vector<std::string> shards;
    DIR* d = opendir(in_dir.c_str());
    if (!d) throw Error("cannot read " + in_dir);
    while (const dirent* e = readdir(d)) {
        const std::string name = e->d_name;
        if (name == "." || name == "..") continue;
        struct stat sb;
        if (stat((in_dir + "/" + name).c_str(), &sb) != 0 || !S_ISREG(sb.st_mode)) continue;
        if (ends_with(name, ".safetensors")) {
            if (name.find("_passthrough") == std::string::npos) shards.push_back(name);
            continue;
        }
        // config, tokenizer, generation settings: copied (:28-34)
        std::string bytes = read_file(in_dir + "/" + name);
        if (name == "config.json") bytes = strip_quantization_config(std::move(bytes));
        write_file(out_dir + "/" + name, bytes);
    }
    closedir(d);
    std::sort(shards.begin(), shards.end());
    for (const std::string& f : shards) dequant_shard(in_dir, f, out_dir);
}

}  // namespace

extern "C" {

tq_model_t tq_model_load(const char* model_path) {
    if (!model_path) return nullptr;
    struct stat sb;
    if (stat(model_path, &sb) != 0 || !S_ISDIR(sb.st_mode)) {
        tq::set_last_error("tq_model_load: not a model directory");
        return nullptr;
    }
    std::unique_ptr<tq_model_s> model;
    try {
        model.reset(new tq_model_s());
        model->path = model_path;
        std::vector<std::string> files;
        if (DIR* d = opendir(model_path)) {
            while (const dirent* e = readdir(d)) {
                const std::string name = e->d_name;
                if (ends_with(name, ".safetensors") && name.find("_passthrough") == std::string::npos) files.push_back(name);
            }
            closedir(d);
        }
        std::sort(files.begin(), files.end());
        for (const std::string& f : files) load_shard(model->path + "/" + f, *model);
        return model.release();
    } catch (const std::exception& e) {
        tq::set_last_error(std::string("tq_model_load: ") + e.what());
        return nullptr;
    } catch (...) {
        tq::set_last_error("tq_model_load: unknown error");
        return nullptr;
    }
}

void* tq_model_forward(tq_model_t, const void*) { return nullptr; }   // a stub in the reference too (src/turboquant_c.cpp:71-77)
void tq_model_free(tq_model_t model) { delete model; }

int tq_model_layer_count(tq_model_t model) { return model ? static_cast<int>(model->layers.size()) : 0; }

const char* tq_model_layer_name(tq_model_t model, int index) {
    if (!model || index < 0 || index >= static_cast<int>(model->names.size())) return nullptr;
    return model->names[static_cast<size_t>(index)].c_str();
}

tq_linear_t tq_model_layer(tq_model_t model, const char* name) {
    if (!model || !name) return nullptr;
    for (size_t i = 0; i < model->names.size(); ++i)
        if (model->names[i] == name) return model->layers[i];
    tq::set_last_error(std::string("tq_model_layer: no quantised layer named ") + name);
    return nullptr;
}

int tq_model_dequant(const char* tq_model_path, const char* output_path) {
    // src/turboquant_c_dequant.cpp:20-191: 0 on success, 1 on any failure.
    if (!tq_model_path || !output_path) return 1;
    try {
        struct stat sb;
        if (stat(tq_model_path, &sb) != 0 || !S_ISDIR(sb.st_mode)) throw Error("not a model directory");
        dequant_model_dir(tq_model_path, output_path);
        return 0;
    } catch (const std::exception& e) {
        tq::set_last_error(std::string("tq_model_dequant: ") + e.what());
    } catch (...) {
        tq::set_last_error("tq_model_dequant: unknown error");
    }
    return 1;
}

}  // extern "C"
