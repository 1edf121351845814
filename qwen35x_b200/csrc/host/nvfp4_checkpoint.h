// On-disk side of the NVFP4 projection path: a safetensors reader and the ModelOpt NVFP4 checkpoint rules.
//
// Mirrors the reference's SafetensorLoader (include/qwen35x/weights/safetensors.h:9-49: resolve_tensor_file,
// load_tensor_info, raw reads) and validate_modelopt_nvfp4_checkpoint (src/weights/modelopt_nvfp4.cpp:147-193) with the
// same `bool` + `std::string & error_message` convention and the same messages, so that the command line's
// --hf-model-dir / --nvfp4-tensor flags take a real checkpoint directory.  Host code only: nothing here touches the GPU.
//
// A tensor family of one quantised linear layer `<base>`:
//   <base>.weight          U8       [N, K/2]   two E2M1 codes per byte, element 2j in the low nibble
//   <base>.weight_scale    F8_E4M3  [N, K/16]  one scale per 16 elements
//   <base>.weight_scale_2  F32      []         per-tensor scale
//   <base>.input_scale     F32      []         activation scale
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace q35b::checkpoint {

struct TensorInfo {
  std::string name;
  std::string dtype;                 // safetensors dtype string: "U8", "F8_E4M3", "F32", "BF16", ...
  std::vector<std::int64_t> shape;   // empty = scalar
  std::uint64_t data_start = 0;      // byte offsets inside the file's data section
  std::uint64_t data_end = 0;
  std::uint64_t data_section = 0;    // file offset of the data section (8 + header length)
};

// The file that holds `tensor_name`: the shard named by model.safetensors.index.json, or, without an index, the
// first *.safetensors file of the directory in name order.
bool resolve_tensor_file(const std::string & model_dir, const std::string & tensor_name, std::string & out_file,
                         std::string & error_message);

// Header entry of one tensor.
bool load_tensor_info(const std::string & safetensors_file, const std::string & tensor_name, TensorInfo & out_info,
                      std::string & error_message);

// Names of all tensors of a file, in header order.
bool list_tensor_names(const std::string & safetensors_file, std::vector<std::string> & names, std::string & error_message);

// Raw bytes of a tensor whose dtype must equal `expected_dtype`.
bool read_tensor_bytes(const std::string & model_dir, const std::string & tensor_name, const std::string & expected_dtype,
                       TensorInfo & info, std::vector<std::uint8_t> & data, std::string & error_message);

bool read_scalar_f32(const std::string & model_dir, const std::string & tensor_name, float & value,
                     std::string & error_message);

struct Nvfp4Tensor {
  std::string base_name;
  int rows = 0;
  int cols = 0;
  std::vector<std::uint8_t> packed_weights;  // [rows, cols / 2]
  std::vector<std::uint8_t> weight_scales;   // [rows, cols / 16]
  float weight_scale_2 = 1.0f;
  float input_scale = 1.0f;
};

// Loads one family and applies the shape / dtype rules below to it.
bool load_nvfp4_tensor(const std::string & model_dir, const std::string & base_name, Nvfp4Tensor & out,
                       std::string & error_message);

struct TensorReport {
  std::string base_name;
  std::vector<std::int64_t> source_shape;  // [N, K]
  std::vector<std::int64_t> packed_shape;  // [N, K/2]
  std::vector<std::int64_t> scale_shape;   // [N, K/16]
};

struct ValidationResult {
  int group_size = 0;
  int quantized_tensors = 0;
  int packed_u8_tensors = 0;
  int fp8_scale_tensors = 0;
  int f32_input_scale_tensors = 0;
  int f32_weight_scale2_tensors = 0;
  std::vector<TensorReport> tensors;
};

// hf_quant_config.json must declare quant_algo NVFP4, group_size 16 and a null kv_cache_quant_algo; every family in
// `base_names` must follow the dtype and shape rules (U8 2-D weight, F8_E4M3 scale of shape [N, K/16], scalar F32
// input_scale and weight_scale_2).  With an empty `base_names` the families are discovered: every tensor named
// `<base>.weight_scale` in the directory's files.
bool validate_nvfp4_checkpoint(const std::string & model_dir, const std::vector<std::string> & base_names,
                               ValidationResult & result, std::string & error_message);

// The module bases the reference expects for a Qwen3.5 text model with `num_layers` layers, where layer i uses full
// attention when (i + 1) % full_attention_interval == 0 and the gated-delta linear attention otherwise
// (src/weights/modelopt_nvfp4.cpp:30-56).
std::vector<std::string> expected_module_bases(int num_layers, int full_attention_interval);

}  // namespace q35b::checkpoint
