// On-disk archive of quantized linear weights, compatible with kmll's export directory:
//   manifest.json                       "quantization": "row-symmetric-int8-with-f32-row-scales"
//   NNNN_<name>.i8  + NNNN_<name>.scales.f32     one pair per tensor, raw little-endian bytes
// (file naming crates/inference/src/rowwise_scaled.rs:141-157; reader :94-106, :159-178; writer
// src/main.rs:5658-5711, :5948-5961; tensor order crates/inference/src/model.rs:9082-9140, index = 1 + layer * 7 +
// offset with 0 = output.weight, :9185-9187; validation by byte length and manifest key :8984-9069).
// W4-G128 archives use the same scheme with a sibling manifest value and the suffixes .w4 / .gscales.f16.
// Host code only (no kernel in this file); tensors pass through kmll_decoder_set_tensor / get_tensor.
#include <sys/stat.h>

#include <cerrno>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/kmll_b200_runtime.h"
#include "common.cuh"

namespace kmll {

static const char* kManifestI8 = "row-symmetric-int8-with-f32-row-scales";
static const char* kManifestW4 = "group128-symmetric-int4-with-f16-group-scales";

// rowwise_scaled_i8_export_file_stem: every character that is not ASCII alphanumeric becomes '_'
static std::string file_stem(const char* name) {
    std::string s(name);
    for (char& ch : s) {
        const bool alnum = (ch >= '0' && ch <= '9') || (ch >= 'a' && ch <= 'z') || (ch >= 'A' && ch <= 'Z');
        if (!alnum) ch = '_';
    }
    return s;
}

static void tensor_paths(const char* dir, int index, const char* name, int format, std::string* values, std::string* scales) {
    char prefix[16];
    snprintf(prefix, sizeof(prefix), "%04d_", index);
    const std::string stem = std::string(dir) + "/" + prefix + file_stem(name);
    *values = stem + (format == KMLL_FORMAT_W4G128 ? ".w4" : ".i8");
    *scales = stem + (format == KMLL_FORMAT_W4G128 ? ".gscales.f16" : ".scales.f32");
}

static bool tensor_bytes(int format, int rows, int cols, size_t* values, size_t* scales) {
    if (rows <= 0 || cols <= 0) return false;
    if (format == KMLL_FORMAT_W4G128) {
        if (cols % 128 != 0) return false;
        *values = (size_t)rows * cols / 2;
        *scales = (size_t)rows * (cols / 128) * 2;
    } else {
        *values = (size_t)rows * cols;
        *scales = (size_t)rows * 4;
    }
    return true;
}

// validate_export_regular_file_len (crates/inference/src/model.rs:9155-9183)
static int check_regular_file(const std::string& path, long long expected_bytes, const char* what) {
    struct stat st;
    if (stat(path.c_str(), &st) != 0) return fail(KMLL_ERR_STATE, "%s %s is not readable: %s", what, path.c_str(), strerror(errno));
    if (!S_ISREG(st.st_mode)) return fail(KMLL_ERR_STATE, "%s %s is not a regular file", what, path.c_str());
    if (expected_bytes >= 0 && (long long)st.st_size != expected_bytes)
        return fail(KMLL_ERR_SHAPE, "%s %s has %lld bytes, expected %lld", what, path.c_str(), (long long)st.st_size, expected_bytes);
    return KMLL_OK;
}

static int write_file(const std::string& path, const void* data, size_t bytes) {
    FILE* f = fopen(path.c_str(), "wb");
    if (f == nullptr) return fail(KMLL_ERR_STATE, "cannot create %s: %s", path.c_str(), strerror(errno));
    const size_t n = bytes ? fwrite(data, 1, bytes, f) : 0;
    const int rc = fclose(f);
    if (n != bytes || rc != 0) return fail(KMLL_ERR_STATE, "short write to %s", path.c_str());
    return KMLL_OK;
}

static int read_file(const std::string& path, void* data, size_t bytes) {
    FILE* f = fopen(path.c_str(), "rb");
    if (f == nullptr) return fail(KMLL_ERR_STATE, "cannot open %s: %s", path.c_str(), strerror(errno));
    const size_t n = bytes ? fread(data, 1, bytes, f) : 0;
    fclose(f);
    if (n != bytes) return fail(KMLL_ERR_SHAPE, "short read from %s", path.c_str());
    return KMLL_OK;
}

static void json_string(std::string* out, const std::string& s) {
    out->push_back('"');
    for (char ch : s) {
        if (ch == '"' || ch == '\\') { out->push_back('\\'); out->push_back(ch); }
        else if (ch == '\n') *out += "\\n";
        else out->push_back(ch);
    }
    out->push_back('"');
}

// Value of a top-level string field, found the way kmll finds it (first occurrence of "field", then ':' and a string;
// crates/inference/src/model.rs:11886-11890).
static bool json_string_field(const std::string& json, const char* field, std::string* value) {
    const std::string key = std::string("\"") + field + "\"";
    size_t pos = json.find(key);
    if (pos == std::string::npos) return false;
    pos += key.size();
    while (pos < json.size() && (json[pos] == ' ' || json[pos] == '\t' || json[pos] == '\n' || json[pos] == '\r')) ++pos;
    if (pos >= json.size() || json[pos] != ':') return false;
    ++pos;
    while (pos < json.size() && (json[pos] == ' ' || json[pos] == '\t' || json[pos] == '\n' || json[pos] == '\r')) ++pos;
    if (pos >= json.size() || json[pos] != '"') return false;
    ++pos;
    value->clear();
    while (pos < json.size() && json[pos] != '"') {
        if (json[pos] == '\\' && pos + 1 < json.size()) ++pos;
        value->push_back(json[pos++]);
    }
    return pos < json.size();
}

struct TensorSpec { int layer, tensor, index, rows, cols; std::string name; };

// all_linear_int8_export_tensor_specs (crates/inference/src/model.rs:9082-9140)
static std::vector<TensorSpec> tensor_specs(const kmll_decoder_config& c) {
    const int q_len = c.n_heads * c.head_dim, kv_len = c.n_kv_heads * c.head_dim;
    std::vector<TensorSpec> specs;
    specs.push_back({-1, KMLL_T_OUTPUT, 0, c.vocab_size, c.dim, "output.weight"});
    const struct { int tensor; const char* name; int rows, cols; } per_layer[7] = {
        {KMLL_T_WQ, "attention.wq.weight", q_len, c.dim},          {KMLL_T_WK, "attention.wk.weight", kv_len, c.dim},
        {KMLL_T_WV, "attention.wv.weight", kv_len, c.dim},         {KMLL_T_WO, "attention.wo.weight", c.dim, q_len},
        {KMLL_T_W1, "feed_forward.w1.weight", c.hidden_dim, c.dim}, {KMLL_T_W3, "feed_forward.w3.weight", c.hidden_dim, c.dim},
        {KMLL_T_W2, "feed_forward.w2.weight", c.dim, c.hidden_dim}};
    for (int l = 0; l < c.n_layers; ++l)
        for (int o = 0; o < 7; ++o)
            specs.push_back({l, per_layer[o].tensor, 1 + l * 7 + o, per_layer[o].rows, per_layer[o].cols,
                             "layers." + std::to_string(l) + "." + per_layer[o].name});
    return specs;
}

}  // namespace kmll

using namespace kmll;

extern "C" {

int kmll_archive_tensor_index(int layer, int offset) {
    if (layer < 0) return 0;
    return 1 + layer * 7 + offset;
}

int kmll_archive_file_paths(const char* dir, int index, const char* name, int format, char* values_path, char* scales_path, size_t capacity) {
    KMLL_REQUIRE_PTR(dir); KMLL_REQUIRE_PTR(name); KMLL_REQUIRE_PTR(values_path); KMLL_REQUIRE_PTR(scales_path);
    std::string v, s;
    tensor_paths(dir, index, name, format, &v, &s);
    if (v.size() + 1 > capacity || s.size() + 1 > capacity) return fail(KMLL_ERR_CAPACITY, "archive path longer than %zu bytes", capacity);
    memcpy(values_path, v.c_str(), v.size() + 1);
    memcpy(scales_path, s.c_str(), s.size() + 1);
    return KMLL_OK;
}

int kmll_archive_write_tensor(const char* dir, int index, const char* name, int format, int rows, int cols, const void* values,
                              const void* scales) {
    KMLL_REQUIRE_PTR(dir); KMLL_REQUIRE_PTR(name); KMLL_REQUIRE_PTR(values); KMLL_REQUIRE_PTR(scales);
    size_t vb = 0, sb = 0;
    if (!tensor_bytes(format, rows, cols, &vb, &sb)) return fail(KMLL_ERR_SHAPE, "archive tensor %s: bad shape %d x %d", name, rows, cols);
    mkdir(dir, 0777);  // (fails harmlessly when the directory exists)
    std::string vp, sp;
    tensor_paths(dir, index, name, format, &vp, &sp);
    int rc = write_file(vp, values, vb);
    if (rc != KMLL_OK) return rc;
    return write_file(sp, scales, sb);
}

// RowwiseScaledI8Matrix::read_exported + from_i8_rows_symmetric_parts: the byte counts must match rows x cols
int kmll_archive_read_tensor(const char* dir, int index, const char* name, int format, int rows, int cols, void* values, void* scales) {
    KMLL_REQUIRE_PTR(dir); KMLL_REQUIRE_PTR(name); KMLL_REQUIRE_PTR(values); KMLL_REQUIRE_PTR(scales);
    size_t vb = 0, sb = 0;
    if (!tensor_bytes(format, rows, cols, &vb, &sb)) return fail(KMLL_ERR_SHAPE, "archive tensor %s: bad shape %d x %d", name, rows, cols);
    std::string vp, sp;
    tensor_paths(dir, index, name, format, &vp, &sp);
    int rc = check_regular_file(vp, (long long)vb, "archive values file");
    if (rc != KMLL_OK) return rc;
    rc = check_regular_file(sp, (long long)sb, "archive scales file");
    if (rc != KMLL_OK) return rc;
    rc = read_file(vp, values, vb);
    if (rc != KMLL_OK) return rc;
    return read_file(sp, scales, sb);
}

int kmll_archive_write_manifest(const char* dir, const kmll_decoder_config* config, const char* weights_path) {
    KMLL_REQUIRE_PTR(dir); KMLL_REQUIRE_PTR(config);
    const std::vector<TensorSpec> specs = tensor_specs(*config);
    std::string out = "{\n  \"model_dir\": ";
    json_string(&out, weights_path ? weights_path : "");
    out += ",\n  \"weights_path\": ";
    json_string(&out, weights_path ? weights_path : "");
    out += ",\n  \"output_dir\": ";
    json_string(&out, dir);
    out += ",\n  \"quantization\": ";
    json_string(&out, config->format == KMLL_FORMAT_W4G128 ? kManifestW4 : kManifestI8);
    out += ",\n  \"planned_tensor_count\": " + std::to_string(specs.size());
    out += ",\n  \"exported_tensor_count\": " + std::to_string(specs.size());
    out += ",\n  \"complete_export\": true,\n  \"tensors\": [\n";
    for (size_t i = 0; i < specs.size(); ++i) {
        const TensorSpec& t = specs[i];
        size_t vb = 0, sb = 0;
        tensor_bytes(config->format, t.rows, t.cols, &vb, &sb);
        std::string vp, sp;
        tensor_paths(dir, t.index, t.name.c_str(), config->format, &vp, &sp);
        out += "    {\"index\": " + std::to_string(t.index) + ", \"name\": ";
        json_string(&out, t.name);
        out += ", \"role\": \"linear\", \"shape\": [" + std::to_string(t.rows) + ", " + std::to_string(t.cols) + "], \"rows\": " + std::to_string(t.rows) +
               ", \"cols\": " + std::to_string(t.cols) + ", \"values_bytes\": " + std::to_string(vb) + ", \"scales_bytes\": " + std::to_string(sb) +
               ", \"values_path\": ";
        json_string(&out, vp);
        out += ", \"scales_path\": ";
        json_string(&out, sp);
        out += i + 1 < specs.size() ? "},\n" : "}\n";
    }
    out += "  ]\n}\n";
    mkdir(dir, 0777);
    return write_file(std::string(dir) + "/manifest.json", out.data(), out.size());
}

// validate_all_linear_int8_export_archive (crates/inference/src/model.rs:8984-9035)
int kmll_archive_validate(const char* dir, const kmll_decoder_config* config, const char* expected_weights_path) {
    KMLL_REQUIRE_PTR(dir); KMLL_REQUIRE_PTR(config);
    struct stat st;
    if (stat(dir, &st) != 0) return fail(KMLL_ERR_STATE, "export directory %s is not readable: %s", dir, strerror(errno));
    if (!S_ISDIR(st.st_mode)) return fail(KMLL_ERR_STATE, "export path %s is not a directory", dir);
    const std::string manifest_path = std::string(dir) + "/manifest.json";
    int rc = check_regular_file(manifest_path, -1, "export manifest");
    if (rc != KMLL_OK) return rc;
    std::string manifest;
    {
        FILE* f = fopen(manifest_path.c_str(), "rb");
        if (f == nullptr) return fail(KMLL_ERR_STATE, "export manifest %s is not readable", manifest_path.c_str());
        char buf[4096];
        size_t n;
        while ((n = fread(buf, 1, sizeof(buf), f)) > 0) manifest.append(buf, n);
        fclose(f);
    }
    std::string quantization;
    if (!json_string_field(manifest, "quantization", &quantization)) return fail(KMLL_ERR_SHAPE, "export manifest %s has no quantization field", manifest_path.c_str());
    const char* expected = config->format == KMLL_FORMAT_W4G128 ? kManifestW4 : kManifestI8;
    if (quantization != expected)
        return fail(KMLL_ERR_UNSUPPORTED, "export manifest %s has unsupported quantization \"%s\" (this decoder expects \"%s\")", manifest_path.c_str(),
                    quantization.c_str(), expected);
    if (expected_weights_path != nullptr) {
        std::string wp;
        if (!json_string_field(manifest, "weights_path", &wp) || wp != expected_weights_path)
            return fail(KMLL_ERR_STATE, "export manifest %s was generated from weights_path %s, but the current model weights source is %s; regenerate the export archive",
                        manifest_path.c_str(), wp.c_str(), expected_weights_path);
    }
    for (const TensorSpec& t : tensor_specs(*config)) {
        size_t vb = 0, sb = 0;
        if (!tensor_bytes(config->format, t.rows, t.cols, &vb, &sb)) return fail(KMLL_ERR_SHAPE, "exported tensor %s: bad shape", t.name.c_str());
        std::string vp, sp;
        tensor_paths(dir, t.index, t.name.c_str(), config->format, &vp, &sp);
        rc = check_regular_file(vp, (long long)vb, "export values file");
        if (rc != KMLL_OK) return rc;
        rc = check_regular_file(sp, (long long)sb, "export scales file");
        if (rc != KMLL_OK) return rc;
    }
    return KMLL_OK;
}

int kmll_decoder_export_archive(kmll_decoder_t dec, const kmll_decoder_config* config, const char* dir, const char* weights_path) {
    KMLL_REQUIRE_PTR(dec); KMLL_REQUIRE_PTR(config); KMLL_REQUIRE_PTR(dir);
    if (config->tp_size != 1) return fail(KMLL_ERR_UNSUPPORTED, "export needs the full tensors: use a decoder with tp_size 1");
    for (const TensorSpec& t : tensor_specs(*config)) {
        size_t vb = 0, sb = 0;
        if (!tensor_bytes(config->format, t.rows, t.cols, &vb, &sb)) return fail(KMLL_ERR_SHAPE, "tensor %s: bad shape", t.name.c_str());
        std::vector<unsigned char> values(vb), scales(sb);
        int rc = kmll_decoder_get_tensor(dec, t.layer, t.tensor, values.data(), scales.data());
        if (rc != KMLL_OK) return rc;
        rc = kmll_archive_write_tensor(dir, t.index, t.name.c_str(), config->format, t.rows, t.cols, values.data(), scales.data());
        if (rc != KMLL_OK) return rc;
    }
    return kmll_archive_write_manifest(dir, config, weights_path);
}

// MinistralAllLinearInt8Runtime::new_from_export (crates/inference/src/model.rs:6327-6384): validate, then read and upload
// every linear tensor (every tensor-parallel rank reads the full tensor and keeps its shard)
int kmll_decoder_load_archive(kmll_decoder_t dec, const kmll_decoder_config* config, const char* dir, const char* expected_weights_path) {
    KMLL_REQUIRE_PTR(dec); KMLL_REQUIRE_PTR(config); KMLL_REQUIRE_PTR(dir);
    int rc = kmll_archive_validate(dir, config, expected_weights_path);
    if (rc != KMLL_OK) return rc;
    for (const TensorSpec& t : tensor_specs(*config)) {
        size_t vb = 0, sb = 0;
        tensor_bytes(config->format, t.rows, t.cols, &vb, &sb);
        std::vector<unsigned char> values(vb), scales(sb);
        rc = kmll_archive_read_tensor(dir, t.index, t.name.c_str(), config->format, t.rows, t.cols, values.data(), scales.data());
        if (rc != KMLL_OK) return rc;
        rc = kmll_decoder_set_tensor(dec, t.layer, t.tensor, values.data(), scales.data());
        if (rc != KMLL_OK) return rc;
    }
    return KMLL_OK;
}

}  // extern "C"
