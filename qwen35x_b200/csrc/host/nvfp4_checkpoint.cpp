// Safetensors reader and ModelOpt NVFP4 checkpoint rules (see nvfp4_checkpoint.h).
//
// File format: 8-byte little-endian header length L, L bytes of JSON
//   {"<name>": {"dtype": "...", "shape": [...], "data_offsets": [begin, end]}, ..., "__metadata__": {...}}
// then the data section; offsets are relative to its start.  The header is parsed with a small recursive-descent
// JSON reader (the reference scans for substrings, src/weights/safetensors.cpp:284-376; a real parser gives the same
// answers on well-formed files and an error instead of a wrong offset on odd ones).
#include "nvfp4_checkpoint.h"

#include <algorithm>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <map>
#include <sstream>

namespace q35b::checkpoint {
namespace {

namespace fs = std::filesystem;

// ---- minimal JSON -----------------------------------------------------------------------------------------------
struct Json {
  enum Kind { kNull, kBool, kNumber, kString, kArray, kObject } kind = kNull;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::vector<Json> items;                             // array
  std::vector<std::pair<std::string, Json>> members;   // object, in file order

  const Json * find(const std::string & key) const {
    for (const auto & m : members) {
      if (m.first == key) return &m.second;
    }
    return nullptr;
  }
};

class JsonParser {
 public:
  explicit JsonParser(const std::string & text) : s_(text) {}

  bool parse(Json & out, std::string & error) {
    if (!value(out, 0)) {
      error = "JSON error at byte " + std::to_string(pos_) + ": " + err_;
      return false;
    }
    skip_ws();
    if (pos_ != s_.size()) {
      error = "JSON error at byte " + std::to_string(pos_) + ": trailing characters";
      return false;
    }
    return true;
  }

 private:
  void skip_ws() {
    while (pos_ < s_.size() && (s_[pos_] == ' ' || s_[pos_] == '\t' || s_[pos_] == '\n' || s_[pos_] == '\r')) ++pos_;
  }
  bool fail(const char * what) {
    err_ = what;
    return false;
  }
  bool literal(const char * word) {
    const size_t n = std::strlen(word);
    if (s_.compare(pos_, n, word) != 0) return fail("unknown literal");
    pos_ += n;
    return true;
  }
  bool string(std::string & out) {
    if (pos_ >= s_.size() || s_[pos_] != '"') return fail("expected a string");
    ++pos_;
    out.clear();
    while (pos_ < s_.size()) {
      const char c = s_[pos_++];
      if (c == '"') return true;
      if (c != '\\') {
        out.push_back(c);
        continue;
      }
      if (pos_ >= s_.size()) break;
      const char e = s_[pos_++];
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
          if (pos_ + 4 > s_.size()) return fail("short \\u escape");
          unsigned cp = 0;
          for (int i = 0; i < 4; ++i) {
            const char h = s_[pos_++];
            cp <<= 4;
            if (h >= '0' && h <= '9') cp |= static_cast<unsigned>(h - '0');
            else if (h >= 'a' && h <= 'f') cp |= static_cast<unsigned>(h - 'a' + 10);
            else if (h >= 'A' && h <= 'F') cp |= static_cast<unsigned>(h - 'A' + 10);
            else return fail("bad \\u escape");
          }
          // tensor names are ASCII; other code points are kept as UTF-8 without surrogate pairing
          if (cp < 0x80) {
            out.push_back(static_cast<char>(cp));
          } else if (cp < 0x800) {
            out.push_back(static_cast<char>(0xC0 | (cp >> 6)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
          } else {
            out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
          }
          break;
        }
        default: return fail("bad escape");
      }
    }
    return fail("unterminated string");
  }
  bool value(Json & out, int depth) {
    if (depth > 64) return fail("nesting too deep");
    skip_ws();
    if (pos_ >= s_.size()) return fail("unexpected end");
    const char c = s_[pos_];
    if (c == '{') {
      ++pos_;
      out.kind = Json::kObject;
      skip_ws();
      if (pos_ < s_.size() && s_[pos_] == '}') {
        ++pos_;
        return true;
      }
      for (;;) {
        skip_ws();
        std::string key;
        if (!string(key)) return false;
        skip_ws();
        if (pos_ >= s_.size() || s_[pos_] != ':') return fail("expected ':'");
        ++pos_;
        Json v;
        if (!value(v, depth + 1)) return false;
        out.members.emplace_back(std::move(key), std::move(v));
        skip_ws();
        if (pos_ < s_.size() && s_[pos_] == ',') {
          ++pos_;
          continue;
        }
        if (pos_ < s_.size() && s_[pos_] == '}') {
          ++pos_;
          return true;
        }
        return fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      ++pos_;
      out.kind = Json::kArray;
      skip_ws();
      if (pos_ < s_.size() && s_[pos_] == ']') {
        ++pos_;
        return true;
      }
      for (;;) {
        Json v;
        if (!value(v, depth + 1)) return false;
        out.items.push_back(std::move(v));
        skip_ws();
        if (pos_ < s_.size() && s_[pos_] == ',') {
          ++pos_;
          continue;
        }
        if (pos_ < s_.size() && s_[pos_] == ']') {
          ++pos_;
          return true;
        }
        return fail("expected ',' or ']'");
      }
    }
    if (c == '"') {
      out.kind = Json::kString;
      return string(out.str);
    }
    if (c == 't') {
      out.kind = Json::kBool;
      out.b = true;
      return literal("true");
    }
    if (c == 'f') {
      out.kind = Json::kBool;
      out.b = false;
      return literal("false");
    }
    if (c == 'n') {
      out.kind = Json::kNull;
      return literal("null");
    }
    // number
    const size_t start = pos_;
    while (pos_ < s_.size() && (std::strchr("+-0123456789.eE", s_[pos_]) != nullptr)) ++pos_;
    if (pos_ == start) return fail("unexpected character");
    try {
      out.num = std::stod(s_.substr(start, pos_ - start));
    } catch (...) {
      return fail("bad number");
    }
    out.kind = Json::kNumber;
    return true;
  }

  const std::string & s_;
  size_t pos_ = 0;
  std::string err_;
};

bool read_text_file(const fs::path & path, std::string & text, std::string & error_message) {
  std::ifstream in(path, std::ios::binary);
  if (!in) {
    error_message = "Could not open file: " + path.string();
    return false;
  }
  std::ostringstream buffer;
  buffer << in.rdbuf();
  text = buffer.str();
  return true;
}

// Header of a shard as parsed JSON plus the offset of its data section.
bool read_header(const std::string & file, Json & header, std::uint64_t & data_section, std::string & error_message) {
  std::ifstream in(file, std::ios::binary);
  if (!in) {
    error_message = "Could not open safetensors shard: " + file;
    return false;
  }
  unsigned char len_bytes[8];
  in.read(reinterpret_cast<char *>(len_bytes), 8);
  std::uint64_t header_len = 0;
  for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | len_bytes[i];
  in.seekg(0, std::ios::end);
  const std::uint64_t file_size = static_cast<std::uint64_t>(in.tellg());
  if (!in || header_len == 0 || header_len > file_size - 8) {
    error_message = "Invalid safetensors header length in: " + file;
    return false;
  }
  std::string text(header_len, '\0');
  in.seekg(8, std::ios::beg);
  in.read(text.data(), static_cast<std::streamsize>(header_len));
  if (!in) {
    error_message = "Could not read safetensors header from: " + file;
    return false;
  }
  std::string jerr;
  if (!JsonParser(text).parse(header, jerr) || header.kind != Json::kObject) {
    error_message = "Malformed safetensors header in: " + file + (jerr.empty() ? "" : " (" + jerr + ")");
    return false;
  }
  data_section = 8 + header_len;
  return true;
}

bool entry_to_info(const std::string & file, const std::string & name, const Json & entry, std::uint64_t data_section,
                   TensorInfo & out, std::string & error_message) {
  const Json * dtype = entry.find("dtype");
  const Json * shape = entry.find("shape");
  const Json * offsets = entry.find("data_offsets");
  if (entry.kind != Json::kObject || dtype == nullptr || dtype->kind != Json::kString || shape == nullptr ||
      shape->kind != Json::kArray || offsets == nullptr || offsets->kind != Json::kArray || offsets->items.size() != 2) {
    error_message = "Malformed header entry for tensor '" + name + "' in: " + file;
    return false;
  }
  out.name = name;
  out.dtype = dtype->str;
  out.shape.clear();
  for (const Json & d : shape->items) {
    if (d.kind != Json::kNumber || d.num < 0) {
      error_message = "Malformed shape for tensor '" + name + "' in: " + file;
      return false;
    }
    out.shape.push_back(static_cast<std::int64_t>(d.num));
  }
  out.data_start = static_cast<std::uint64_t>(offsets->items[0].num);
  out.data_end = static_cast<std::uint64_t>(offsets->items[1].num);
  out.data_section = data_section;
  if (out.data_end < out.data_start) {
    error_message = "Malformed data_offsets for tensor '" + name + "' in: " + file;
    return false;
  }
  return true;
}

std::vector<std::string> shard_files(const fs::path & root) {
  std::vector<std::string> files;
  std::error_code ec;
  for (const auto & e : fs::directory_iterator(root, ec)) {
    if (e.is_regular_file() && e.path().extension() == ".safetensors") files.push_back(e.path().string());
  }
  std::sort(files.begin(), files.end());
  return files;
}

std::string shape_string(const std::vector<std::int64_t> & shape) {
  std::ostringstream out;
  out << "[";
  for (size_t i = 0; i < shape.size(); ++i) out << (i ? "," : "") << shape[i];
  out << "]";
  return out.str();
}

bool load_info_from_dir(const std::string & model_dir, const std::string & name, TensorInfo & info, std::string & file,
                        std::string & error_message) {
  return resolve_tensor_file(model_dir, name, file, error_message) && load_tensor_info(file, name, info, error_message);
}

// dtype and shape rules of one family (src/weights/modelopt_nvfp4.cpp:88-145)
bool check_family(const std::string & base_name, int group_size, const TensorInfo & weight, const TensorInfo & scale,
                  const TensorInfo & input_scale, const TensorInfo & weight_scale_2, TensorReport & report,
                  std::string & error_message) {
  if (weight.dtype != "U8") {
    error_message = "Tensor '" + weight.name + "' has dtype " + weight.dtype + " (expected U8).";
    return false;
  }
  if (scale.dtype != "F8_E4M3") {
    error_message = "Tensor '" + scale.name + "' has dtype " + scale.dtype + " (expected F8_E4M3).";
    return false;
  }
  if (input_scale.dtype != "F32" || !input_scale.shape.empty()) {
    error_message = "Tensor '" + input_scale.name + "' must be scalar F32.";
    return false;
  }
  if (weight_scale_2.dtype != "F32" || !weight_scale_2.shape.empty()) {
    error_message = "Tensor '" + weight_scale_2.name + "' must be scalar F32.";
    return false;
  }
  if (weight.shape.size() != 2 || scale.shape.size() != 2) {
    error_message = "NVFP4 tensors for '" + base_name + "' must be 2D.";
    return false;
  }
  if ((weight.shape[1] * 2) % group_size != 0) {
    error_message = "Packed tensor '" + weight.name + "' has an invalid column count for group_size.";
    return false;
  }
  const std::vector<std::int64_t> source_shape = {weight.shape[0], weight.shape[1] * 2};
  const std::vector<std::int64_t> expected_scale = {source_shape[0], source_shape[1] / group_size};
  if (scale.shape != expected_scale) {
    error_message = "Tensor '" + scale.name + "' shape " + shape_string(scale.shape) + " does not match expected " +
                    shape_string(expected_scale) + ".";
    return false;
  }
  report.base_name = base_name;
  report.source_shape = source_shape;
  report.packed_shape = weight.shape;
  report.scale_shape = scale.shape;
  return true;
}

bool read_bytes_at(const std::string & file, const TensorInfo & info, std::vector<std::uint8_t> & data,
                   std::string & error_message) {
  std::ifstream in(file, std::ios::binary);
  if (!in) {
    error_message = "Could not open safetensors shard: " + file;
    return false;
  }
  data.resize(static_cast<size_t>(info.data_end - info.data_start));
  in.seekg(static_cast<std::streamoff>(info.data_section + info.data_start), std::ios::beg);
  in.read(reinterpret_cast<char *>(data.data()), static_cast<std::streamsize>(data.size()));
  if (!in) {
    error_message = "Could not read tensor '" + info.name + "' from: " + file;
    return false;
  }
  return true;
}

}  // namespace

bool resolve_tensor_file(const std::string & model_dir, const std::string & tensor_name, std::string & out_file,
                         std::string & error_message) {
  const fs::path root(model_dir);
  std::error_code ec;
  if (!fs::exists(root, ec) || !fs::is_directory(root, ec)) {
    error_message = "Model directory does not exist: " + model_dir;
    return false;
  }
  const fs::path index_path = root / "model.safetensors.index.json";
  if (!fs::is_regular_file(index_path, ec)) {
    const auto files = shard_files(root);
    if (!files.empty()) {
      out_file = files.front();
      return true;
    }
    error_message = "No safetensors index or shard files found in: " + model_dir;
    return false;
  }
  std::string text;
  if (!read_text_file(index_path, text, error_message)) return false;
  Json index;
  std::string jerr;
  if (!JsonParser(text).parse(index, jerr) || index.kind != Json::kObject) {
    error_message = "Malformed model.safetensors.index.json in: " + model_dir;
    return false;
  }
  const Json * map = index.find("weight_map");
  const Json * shard = (map != nullptr && map->kind == Json::kObject) ? map->find(tensor_name) : nullptr;
  if (shard == nullptr || shard->kind != Json::kString) {
    error_message = "Tensor '" + tensor_name + "' not found in model.safetensors.index.json";
    return false;
  }
  const fs::path shard_path = root / shard->str;
  if (!fs::is_regular_file(shard_path, ec)) {
    error_message = "Indexed shard file does not exist: " + shard_path.string();
    return false;
  }
  out_file = shard_path.string();
  return true;
}

bool load_tensor_info(const std::string & safetensors_file, const std::string & tensor_name, TensorInfo & out_info,
                      std::string & error_message) {
  Json header;
  std::uint64_t data_section = 0;
  if (!read_header(safetensors_file, header, data_section, error_message)) return false;
  const Json * entry = tensor_name == "__metadata__" ? nullptr : header.find(tensor_name);
  if (entry == nullptr) {
    error_message = "Tensor '" + tensor_name + "' not found in: " + safetensors_file;
    return false;
  }
  return entry_to_info(safetensors_file, tensor_name, *entry, data_section, out_info, error_message);
}

bool list_tensor_names(const std::string & safetensors_file, std::vector<std::string> & names, std::string & error_message) {
  Json header;
  std::uint64_t data_section = 0;
  if (!read_header(safetensors_file, header, data_section, error_message)) return false;
  names.clear();
  for (const auto & m : header.members) {
    if (m.first != "__metadata__") names.push_back(m.first);
  }
  return true;
}

bool read_tensor_bytes(const std::string & model_dir, const std::string & tensor_name, const std::string & expected_dtype,
                       TensorInfo & info, std::vector<std::uint8_t> & data, std::string & error_message) {
  std::string file;
  if (!load_info_from_dir(model_dir, tensor_name, info, file, error_message)) return false;
  if (info.dtype != expected_dtype) {
    error_message = "Tensor '" + tensor_name + "' has dtype " + info.dtype + " (expected " + expected_dtype + ").";
    return false;
  }
  return read_bytes_at(file, info, data, error_message);
}

bool read_scalar_f32(const std::string & model_dir, const std::string & tensor_name, float & value,
                     std::string & error_message) {
  TensorInfo info;
  std::vector<std::uint8_t> data;
  if (!read_tensor_bytes(model_dir, tensor_name, "F32", info, data, error_message)) return false;
  if (!info.shape.empty() || data.size() != 4) {
    error_message = "Tensor '" + tensor_name + "' must be scalar F32.";
    return false;
  }
  std::memcpy(&value, data.data(), 4);
  return true;
}

bool load_nvfp4_tensor(const std::string & model_dir, const std::string & base_name, Nvfp4Tensor & out,
                       std::string & error_message) {
  TensorInfo weight, scale, in_scale, s2;
  std::string file;
  if (!read_tensor_bytes(model_dir, base_name + ".weight", "U8", weight, out.packed_weights, error_message) ||
      !read_tensor_bytes(model_dir, base_name + ".weight_scale", "F8_E4M3", scale, out.weight_scales, error_message) ||
      !load_info_from_dir(model_dir, base_name + ".input_scale", in_scale, file, error_message) ||
      !load_info_from_dir(model_dir, base_name + ".weight_scale_2", s2, file, error_message)) {
    return false;
  }
  TensorReport report;
  if (!check_family(base_name, 16, weight, scale, in_scale, s2, report, error_message)) return false;
  if (!read_scalar_f32(model_dir, base_name + ".input_scale", out.input_scale, error_message) ||
      !read_scalar_f32(model_dir, base_name + ".weight_scale_2", out.weight_scale_2, error_message)) {
    return false;
  }
  out.base_name = base_name;
  out.rows = static_cast<int>(report.source_shape[0]);
  out.cols = static_cast<int>(report.source_shape[1]);
  if (out.packed_weights.size() != static_cast<size_t>(out.rows) * (out.cols / 2) ||
      out.weight_scales.size() != static_cast<size_t>(out.rows) * (out.cols / 16)) {
    error_message = "NVFP4 packed weight or scale size does not match matrix dimensions.";
    return false;
  }
  return true;
}

bool validate_nvfp4_checkpoint(const std::string & model_dir, const std::vector<std::string> & base_names,
                               ValidationResult & result, std::string & error_message) {
  if (model_dir.empty()) {
    error_message = "model_dir is required for ModelOpt NVFP4 validation.";
    return false;
  }
  const fs::path root(model_dir);
  std::string text;
  if (!read_text_file(root / "hf_quant_config.json", text, error_message)) return false;
  Json config;
  std::string jerr;
  if (!JsonParser(text).parse(config, jerr) || config.kind != Json::kObject) {
    error_message = "Malformed hf_quant_config.json in: " + model_dir;
    return false;
  }
  // {"quantization": {"quant_algo": "NVFP4", "kv_cache_quant_algo": null, "group_size": 16, ...}} (keys may also sit
  // at the top level)
  const Json * q = config.find("quantization");
  if (q == nullptr || q->kind != Json::kObject) q = &config;
  const Json * algo = q->find("quant_algo");
  if (algo == nullptr || algo->kind != Json::kString || algo->str != "NVFP4") {
    error_message = "hf_quant_config.json does not declare quant_algo=NVFP4.";
    return false;
  }
  const Json * group = q->find("group_size");
  if (group == nullptr || group->kind != Json::kNumber || group->num != 16.0) {
    error_message = "hf_quant_config.json does not declare group_size=16.";
    return false;
  }
  const Json * kv = q->find("kv_cache_quant_algo");
  if (kv == nullptr || kv->kind != Json::kNull) {
    error_message = "hf_quant_config.json must leave kv_cache_quant_algo null for the current plan.";
    return false;
  }

  std::vector<std::string> bases = base_names;
  if (bases.empty()) {
    const std::string suffix = ".weight_scale";
    for (const std::string & file : shard_files(root)) {
      std::vector<std::string> names;
      if (!list_tensor_names(file, names, error_message)) return false;
      for (const std::string & n : names) {
        if (n.size() > suffix.size() && n.compare(n.size() - suffix.size(), suffix.size(), suffix) == 0) {
          bases.push_back(n.substr(0, n.size() - suffix.size()));
        }
      }
    }
    std::sort(bases.begin(), bases.end());
    if (bases.empty()) {
      error_message = "No NVFP4 tensor families found in: " + model_dir;
      return false;
    }
  }

  result = {};
  result.group_size = 16;
  for (const std::string & base : bases) {
    TensorInfo weight, scale, in_scale, s2;
    std::string file;
    if (!load_info_from_dir(model_dir, base + ".weight", weight, file, error_message) ||
        !load_info_from_dir(model_dir, base + ".weight_scale", scale, file, error_message) ||
        !load_info_from_dir(model_dir, base + ".input_scale", in_scale, file, error_message) ||
        !load_info_from_dir(model_dir, base + ".weight_scale_2", s2, file, error_message)) {
      return false;
    }
    TensorReport report;
    if (!check_family(base, result.group_size, weight, scale, in_scale, s2, report, error_message)) return false;
    result.tensors.push_back(std::move(report));
  }
  result.quantized_tensors = static_cast<int>(result.tensors.size());
  result.packed_u8_tensors = result.quantized_tensors;
  result.fp8_scale_tensors = result.quantized_tensors;
  result.f32_input_scale_tensors = result.quantized_tensors;
  result.f32_weight_scale2_tensors = result.quantized_tensors;
  return true;
}

std::vector<std::string> expected_module_bases(int num_layers, int full_attention_interval) {
  std::vector<std::string> names;
  for (int layer = 0; layer < num_layers; ++layer) {
    const std::string base = "model.language_model.layers." + std::to_string(layer) + ".";
    names.push_back(base + "mlp.gate_proj");
    names.push_back(base + "mlp.up_proj");
    names.push_back(base + "mlp.down_proj");
    const bool full = full_attention_interval > 0 && (layer + 1) % full_attention_interval == 0;
    if (full) {
      for (const char * p : {"self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj"}) names.push_back(base + p);
    } else {
      for (const char * p : {"linear_attn.in_proj_qkv", "linear_attn.in_proj_z", "linear_attn.in_proj_b", "linear_attn.in_proj_a",
                             "linear_attn.out_proj"}) {
        names.push_back(base + p);
      }
    }
  }
  return names;
}

}  // namespace q35b::checkpoint
