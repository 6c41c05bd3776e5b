"""Wire-format declaration of the TTNN flatbuffer, restricted to what the B200 runtime reads.

Source of truth for field order (field ids are positional) are the reference's
schema files under include/ttmlir/Target/:
  Common/types.fbs, Common/version.fbs, Common/debug_info.fbs,
  TTNN/types.fbs, TTNN/program.fbs, TTNN/binary.fbs, TTNN/operations/*.fbs.
Every table the runtime touches lists ALL of its fields so that the ids line up;
fields whose payload the runtime never looks at (TT-specific program configs,
shard specs, core grids) are declared `opaque` / `opaque_union`: they occupy
their slot(s) but get no accessor.  Tables of ops outside the supported set are
not declared at all; they only appear as names in the `OpType` union so that
the union's type ids are right and the executor can name what it rejects.

Both the Python emitter (schema/fbs.py Writer) and the generated C++ accessors
(runtime/generated/ttnn_schema.h, made by schema/gen_cpp.py) come from this one
declaration.
"""

from .fbs import OPT, Schema

S = Schema()

# ------------------------------------------------------------------ tt.target
S.namespace("tt::target")

S.struct("Dim2d", [("y", "i32"), ("x", "i32")])
S.struct("Version", [("major", "u16"), ("minor", "u16"), ("patch", "u32")])

S.enum("Arch", "u32", ["Wormhole_b0", "Blackhole", "Quasar"])
S.enum("DataType", "u16", [
    "Float32", "Float16", "BFloat16", "BFP_Float8", "BFP_BFloat8", "BFP_Float4", "BFP_BFloat4",
    "BFP_Float2", "BFP_BFloat2", "UInt32", "UInt16", "UInt8", "Int32",
    "Float64", "Int64", "UInt64", "Int16", "Int8", "Bool"])
S.enum("OOBVal", "u16", ["Undef", "Zero", "One", "Inf", "NegInf"])
S.enum("TensorLayout", "u16", ["RowMajor", "Tile", "Invalid"])
S.enum("BufferType", "u16", ["DRAM", "L1", "SystemMemory", "L1Small", "Trace"])
S.enum("CPURole", "u8", ["Host", "Device"])
S.enum("MathFidelity", "u8", {"LoFi": 0, "HiFi2": 2, "HiFi3": 3, "HiFi4": 4})
S.enum("MeshShardDirection", "u32", ["FullToShardShape", "ShardToFullShape"])
S.enum("MeshShardType", "u32", ["Replicate", "Maximal", "Devices"])
S.enum("Topology", "u16", ["Ring", "Linear", "Mesh", "Torus"])

S.struct("ChipCoord", [("rack", "u32"), ("shelf", "u32"), ("y", "u32"), ("x", "u32")])

S.table("ChipDesc", [
    ("arch", "Arch"), ("grid_size", "Dim2d"), ("coord_translation_offsets", "Dim2d"),
    ("l1_size", "u64"), ("num_dram_channels", "u32"), ("dram_channel_size", "u64"),
    ("noc_l1_address_align_bytes", "u32"), ("pcie_address_align_bytes", "u32"),
    ("noc_dram_address_align_bytes", "u32"), ("l1_unreserved_base", "u32"),
    ("erisc_l1_unreserved_base", "u32"), ("dram_unreserved_base", "u32"),
    ("dram_unreserved_end", "u32"), ("supported_data_types", "[DataType]"),
    ("supported_tile_sizes", "[Dim2d]"), ("dst_physical_size_tiles", "u32"),
    ("num_cbs", "u32"), ("num_compute_threads", "u32"), ("num_datamovement_threads", "u32"),
    ("dram_grid_size", "Dim2d"), ("dram_bank_to_logical_worker_noc0", "[Dim2d]"),
    ("dram_bank_to_logical_worker_noc1", "[Dim2d]"),
])
S.table("CPUDesc", [("role", "CPURole"), ("target_triple", "string")])
S.table("SystemDesc", [
    ("cpu_descs", "[CPUDesc]"), ("chip_descs", "[ChipDesc]"), ("chip_desc_indices", "[u32]"),
    ("chip_capabilities", "[u32]"), ("chip_coords", "[ChipCoord]"), ("chip_channels", "opaque"),
])
# Root of a system-descriptor file (identifier "TTSY", Common/system_desc.fbs): what
# getCurrentSystemDesc returns and `ttrt query` stores.
S.table("SystemDescRoot", [
    ("version", "Version"), ("schema_hash", "string"), ("ttmlir_git_hash", "string"),
    ("product_identifier", "string"), ("system_desc", "SystemDesc")])
S.table("DeviceRef", [("global_id", "u32")])
S.table("DynamicLib", [("dylib_id", "u32"), ("raw_file", "[u8]")])
S.table("MLIR", [("name", "string"), ("source", "string")])

S.table("GoldenTensor", [
    ("name", "string"), ("shape", "[i64]"), ("stride", "[i64]"), ("dtype", "DataType"),
    ("data", "[u8]")])
S.table("GoldenDeviceTensor", [("device", "u32"), ("value", "GoldenTensor")])
S.table("GoldenKV", [("key", "string"), ("value", "[GoldenDeviceTensor]")])
S.table("GoldenInfo", [("golden_map", "[GoldenKV]")])
S.table("DebugInfo", [("cpp", "string"), ("mlir_stages", "[MLIR]"), ("golden_info", "GoldenInfo")])

# ------------------------------------------------------------ tt.target.ttnn
S.namespace("tt::target::ttnn")

S.enum("TensorMemoryLayout", "u16",
       ["Interleaved", "HeightSharded", "WidthSharded", "BlockSharded", "NDSharded"])
S.enum("StorageType", "u16", ["Host", "Device"])
S.enum("ShardStatus", "u32", ["Presharded", "Unsharded"])
S.enum("PlacementType", "u16", ["Replicate", "Shard"])
S.struct("Placement", [("type", "PlacementType"), ("dim", "i32")])

S.table("MemoryConfig", [
    ("tensor_memory_layout", "TensorMemoryLayout"), ("buffer_type", "BufferType"),
    ("shard_spec", "opaque"), ("nd_shard_spec", "opaque")])
S.table("MemoryDesc", [
    ("storage_type", "StorageType"), ("tile_shape", "Dim2d"), ("data_type", "DataType"),
    ("memory_config", "MemoryConfig")])
S.table("LayoutDesc", [("oob_val", "OOBVal"), ("memory_desc", "MemoryDesc")])
S.table("TensorDesc", [
    ("shape", "[i32]"), ("mesh_shape", "[i32]"), ("layout", "LayoutDesc"),
    ("shard_status", "ShardStatus"), ("local_shape", "[i32]")])
S.table("TensorRef", [("global_id", "u32"), ("desc", "TensorDesc")])
S.table("GlobalSemaphoreRef", [("global_id", "u32")])
S.table("FloatingPointType", [("value", "f32")])
S.table("IntegralType", [("value", "i32")])
S.union("NumberType", [("FP", "FloatingPointType"), ("I32", "IntegralType")])
S.table("MeshMapperConfig", [("placements", "[Placement]"), ("mesh_shape_override", "[u32]")])
S.table("MeshComposerConfig", [("dims", "[i32]"), ("mesh_shape_override", "[u32]")])

S.table("DeviceComputeKernelConfig", [
    ("math_fidelity", "MathFidelity", OPT), ("math_approx_mode", "bool", OPT),
    ("fp32_dest_acc_en", "bool", OPT), ("packer_l1_acc", "bool", OPT),
    ("dst_full_sync_en", "bool", OPT)])

# --- eltwise (operations/eltwise.fbs)
S.table("EltwiseOpWithFloatParams", [("parameter", "f32")])
S.enum("EltwiseBinaryOpType", "u32", [
    "Add", "Multiply", "LogicalRightShift", "Subtract", "Equal", "NotEqual", "GreaterEqual",
    "GreaterThan", "LessEqual", "LessThan", "Divide", "LogicalAnd", "LogicalOr", "LogicalXor"])
S.table("EltwiseBinaryOp", [
    ("type", "EltwiseBinaryOpType"), ("lhs", "TensorRef"), ("rhs", "TensorRef"),
    ("output_dtype", "DataType", OPT), ("memory_config", "MemoryConfig"), ("out", "TensorRef")])
S.enum("EltwiseBinaryCompositeOpType", "u32", [
    "Maximum", "Minimum", "Remainder", "Pow", "Atan2", "BitwiseAnd", "BitwiseOr", "BitwiseXor",
    "LogicalLeftShift"])
S.table("EltwiseBinaryCompositeOp", [
    ("type", "EltwiseBinaryCompositeOpType"), ("lhs", "TensorRef"), ("rhs", "TensorRef"),
    ("memory_config", "MemoryConfig"), ("out", "TensorRef")])
S.enum("EltwiseQuantizationOpType", "u32", ["Quantize", "Dequantize", "Requantize"])
S.table("PerTensorScale", [("scale", "f32")])
S.table("PerAxisScale", [("scale", "TensorRef")])
S.union("QuantizationScale", ["PerTensorScale", "PerAxisScale"])
S.table("PerTensorZeroPoint", [("zero_point", "i32")])
S.table("PerAxisZeroPoint", [("zero_point", "TensorRef")])
S.union("QuantizationZeroPoint", ["PerTensorZeroPoint", "PerAxisZeroPoint"])
S.table("QuantizeDequantizeOpParams", [
    ("scale", "QuantizationScale"), ("zero_point", "QuantizationZeroPoint")])
S.table("RequantizeOpParams", [
    ("in_scale", "QuantizationScale"), ("in_zero_point", "QuantizationZeroPoint"),
    ("out_scale", "QuantizationScale"), ("out_zero_point", "QuantizationZeroPoint")])
S.union("EltwiseQuantizationOpParams", ["QuantizeDequantizeOpParams", "RequantizeOpParams"])
S.table("EltwiseQuantizationOp", [
    ("type", "EltwiseQuantizationOpType"), ("in", "TensorRef"), ("axis", "i32", OPT),
    ("output_dtype", "DataType", OPT), ("memory_config", "MemoryConfig"), ("out", "TensorRef"),
    ("params", "EltwiseQuantizationOpParams")])
S.table("EltwiseTernaryWhereOp", [
    ("first", "TensorRef"), ("second", "TensorRef"), ("third", "TensorRef"),
    ("memory_config", "MemoryConfig"), ("out", "TensorRef")])
S.enum("EltwiseUnaryOpType", "u32", [
    "Abs", "Ceil", "Cos", "Floor", "Gelu", "IsFinite", "LogicalNot", "Neg", "Relu", "Sqrt",
    "Rsqrt", "Sigmoid", "Sin", "Reciprocal", "Sign", "Tan", "Tanh", "Atan", "Exp", "Erf", "Erfc",
    "Log", "Expm1", "LeakyRelu", "BitwiseNot", "Relu6", "Silu", "Hardsigmoid", "Mish", "Acos",
    "Asin", "Asinh"])
S.union("EltwiseUnaryOpParams", ["EltwiseOpWithFloatParams"])
S.table("EltwiseUnaryOp", [
    ("type", "EltwiseUnaryOpType"), ("in", "TensorRef"), ("memory_config", "MemoryConfig"),
    ("out", "TensorRef"), ("params", "EltwiseUnaryOpParams")])
S.enum("EltwiseUnaryCompositeOpType", "u32", ["Cbrt", "ClampScalar", "ClampTensor", "Log1p"])
S.table("ClampScalarOpParams", [("min", "NumberType"), ("max", "NumberType")])
S.table("ClampTensorOpParams", [("min", "TensorRef"), ("max", "TensorRef")])
S.union("EltwiseUnaryCompositeOpParams", ["ClampScalarOpParams", "ClampTensorOpParams"])
S.table("EltwiseUnaryCompositeOp", [
    ("type", "EltwiseUnaryCompositeOpType"), ("in", "TensorRef"),
    ("memory_config", "MemoryConfig"), ("out", "TensorRef"),
    ("params", "EltwiseUnaryCompositeOpParams")])

# --- matmul (operations/matmul.fbs)
S.table("MatmulOp", [
    ("a", "TensorRef"), ("b", "TensorRef"), ("out", "TensorRef"), ("transpose_a", "bool"),
    ("transpose_b", "bool"), ("matmul_program_config", "opaque_union"), ("activation", "string"),
    ("compute_config", "DeviceComputeKernelConfig")])
S.table("LinearOp", [
    ("a", "TensorRef"), ("b", "TensorRef"), ("bias", "TensorRef"), ("out", "TensorRef"),
    ("transpose_a", "bool"), ("transpose_b", "bool"), ("matmul_program_config", "opaque_union"),
    ("activation", "string"), ("compute_config", "DeviceComputeKernelConfig")])

# --- conv (operations/conv.fbs)
S.table("Conv2dOp", [
    ("input", "TensorRef"), ("weight", "TensorRef"), ("bias", "TensorRef"), ("out", "TensorRef"),
    ("device", "DeviceRef"), ("in_channels", "u32"), ("out_channels", "u32"),
    ("batch_size", "u32"), ("input_height", "u32"), ("input_width", "u32"),
    ("kernel_size", "[i32]"), ("stride", "[i32]"), ("padding", "[i32]"), ("dilation", "[i32]"),
    ("groups", "u32"), ("output_dtype", "DataType", OPT), ("conv2d_config", "opaque"),
    ("compute_config", "DeviceComputeKernelConfig"), ("conv2d_slice_config", "opaque")])

# --- layout (operations/layout.fbs)
S.table("FromDeviceOp", [("in", "TensorRef"), ("out", "TensorRef")])
S.table("ToDeviceOp", [
    ("in", "TensorRef"), ("device", "DeviceRef"), ("memcfg", "MemoryConfig"),
    ("out", "TensorRef")])
S.table("ToLayoutOp", [
    ("in", "TensorRef"), ("layout", "TensorLayout"), ("dtype", "DataType", OPT),
    ("memcfg", "MemoryConfig"), ("out", "TensorRef")])
S.table("ToMemoryConfigOp", [("in0", "TensorRef"), ("memcfg", "MemoryConfig"), ("out", "TensorRef")])
S.table("TypecastOp", [
    ("in", "TensorRef"), ("dtype", "DataType"), ("memcfg", "MemoryConfig"), ("out", "TensorRef")])

# --- creation (operations/creation.fbs)
S.table("ArangeOp", [
    ("device", "DeviceRef"), ("start", "f32"), ("end", "f32"), ("step", "f32"),
    ("dtype", "DataType", OPT), ("layout", "TensorLayout", OPT), ("memcfg", "MemoryConfig"),
    ("out", "TensorRef")])
S.table("ConstantOp", [
    ("device", "DeviceRef"), ("input", "[u8]"), ("input_dtype", "DataType"),
    ("dtype", "DataType", OPT), ("layout", "TensorLayout", OPT), ("memcfg", "MemoryConfig"),
    ("out", "TensorRef")])
S.table("EmptyOp", [
    ("device", "DeviceRef"), ("shape", "[i64]"), ("dtype", "DataType"), ("layout", "TensorLayout"),
    ("memcfg", "MemoryConfig"), ("out", "TensorRef")])
S.table("FullOp", [
    ("device", "DeviceRef"), ("shape", "[i64]"), ("fill_value", "NumberType"),
    ("dtype", "DataType", OPT), ("layout", "TensorLayout", OPT), ("memcfg", "MemoryConfig"),
    ("out", "TensorRef")])
S.enum("NamedFullOpType", "u32", ["Zeros", "Ones"])
S.table("NamedFullOp", [
    ("type", "NamedFullOpType"), ("device", "DeviceRef"), ("shape", "[i64]"),
    ("dtype", "DataType", OPT), ("layout", "TensorLayout", OPT), ("memcfg", "MemoryConfig"),
    ("out", "TensorRef")])

# --- misc single-table files
S.table("DeallocateOp", [("in", "TensorRef"), ("force", "bool")])
S.table("GetDeviceOp", [
    ("mesh", "Dim2d"), ("offset", "Dim2d"), ("chip_ids", "[u32]"), ("out", "DeviceRef")])
S.table("CpuOp", [
    ("ins", "[TensorRef]"), ("outs", "[TensorRef]"), ("func_name", "string"), ("dylib_id", "u32")])

# --- reduction / normalization
S.enum("ReductionOpType", "u32", ["Sum", "Mean", "Max", "Min"])
S.table("ReductionOp", [
    ("type", "ReductionOpType"), ("in", "TensorRef"), ("out", "TensorRef"), ("dim_arg", "[i32]"),
    ("keep_dim", "bool"), ("compute_config", "DeviceComputeKernelConfig")])
S.table("SoftmaxOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("dimension", "i32"),
    ("numeric_stable", "bool"), ("compute_config", "DeviceComputeKernelConfig")])
S.table("RMSNormOp", [
    ("input", "TensorRef"), ("weight", "TensorRef"), ("bias", "TensorRef"), ("epsilon", "f32"),
    ("memory_config", "MemoryConfig"), ("out", "TensorRef"),
    ("compute_config", "DeviceComputeKernelConfig")])

S.table("LayerNormOp", [
    ("input", "TensorRef"), ("weight", "TensorRef"), ("bias", "TensorRef"), ("epsilon", "f32"),
    ("memory_config", "MemoryConfig"), ("out", "TensorRef")])
S.table("ReductionArgMaxOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("dim", "i32", OPT), ("keep_dim", "bool"),
    ("memcfg", "MemoryConfig")])
# operations/cumsum.fbs
S.table("CumSumOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("dim", "i32"), ("dtype", "DataType", OPT),
    ("memcfg", "MemoryConfig")])
# operations/cumprod.fbs, operations/reduction.fbs (prod), operations/normalization.fbs (batch norm),
# operations/pool.fbs (upsample), operations/conv.fbs (weight / bias preparation)
S.table("CumProdOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("dim", "i32"), ("dtype", "DataType", OPT),
    ("memcfg", "MemoryConfig")])
S.table("ReductionProdOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("dim_arg", "i64", OPT), ("keep_dim", "bool"),
    ("memcfg", "MemoryConfig")])
S.table("BatchNormInferenceOp", [
    ("input", "TensorRef"), ("running_mean", "TensorRef"), ("running_var", "TensorRef"), ("epsilon", "f32"),
    ("weight", "TensorRef"), ("bias", "TensorRef"), ("memory_config", "MemoryConfig"), ("out", "TensorRef"),
    ("compute_config", "DeviceComputeKernelConfig")])
S.table("GroupNormOp", [
    ("input", "TensorRef"), ("input_mask", "TensorRef"), ("weight", "TensorRef"), ("bias", "TensorRef"),
    ("num_groups", "i64"), ("epsilon", "f32"), ("memory_config", "MemoryConfig"), ("out", "TensorRef")])
S.table("ConvTranspose2dOp", [
    ("input", "TensorRef"), ("weight", "TensorRef"), ("bias", "TensorRef"), ("out", "TensorRef"),
    ("device", "DeviceRef"), ("in_channels", "u32"), ("out_channels", "u32"), ("batch_size", "u32"),
    ("input_height", "u32"), ("input_width", "u32"), ("kernel_size", "[i32]"), ("stride", "[i32]"),
    ("padding", "[i32]"), ("output_padding", "[i32]"), ("dilation", "[i32]"), ("groups", "u32"),
    ("output_dtype", "DataType", OPT), ("conv2d_config", "opaque"), ("compute_config", "DeviceComputeKernelConfig"),
    ("memory_config", "MemoryConfig"), ("conv2d_slice_config", "opaque")])
S.table("Conv1dOp", [
    ("input", "TensorRef"), ("weight", "TensorRef"), ("bias", "TensorRef"), ("out", "TensorRef"),
    ("device", "DeviceRef"), ("in_channels", "u32"), ("out_channels", "u32"), ("batch_size", "u32"),
    ("input_length", "u32"), ("kernel_size", "u32"), ("stride", "u32"), ("padding", "[i32]"), ("dilation", "u32"),
    ("groups", "u32"), ("output_dtype", "DataType", OPT), ("conv2d_config", "opaque"),
    ("compute_config", "DeviceComputeKernelConfig"), ("conv2d_slice_config", "opaque")])
S.table("BitcastConvertOp", [("in", "TensorRef"), ("dtype", "DataType"), ("memcfg", "MemoryConfig"), ("out", "TensorRef")])
S.table("NLPConcatHeadsOp", [("in", "TensorRef"), ("out", "TensorRef"), ("memcfg", "MemoryConfig")])
S.table("AssignOp", [
    ("input", "TensorRef"), ("output", "TensorRef"), ("output_memory_config", "MemoryConfig"),
    ("output_dtype", "DataType", OPT)])
S.enum("EltwiseBinaryCompositeScalarOpType", "u32", ["PowScalar"])
S.table("EltwiseBinaryCompositeScalarOp", [
    ("type", "EltwiseBinaryCompositeScalarOpType"), ("lhs", "TensorRef"), ("rhs", "NumberType"),
    ("memory_config", "MemoryConfig"), ("out", "TensorRef")])
S.table("DumpTensorOp", [("file_path", "string"), ("in", "TensorRef")])
S.table("LoadTensorOp", [("file_path", "string"), ("device", "DeviceRef"), ("out", "TensorRef")])
S.table("AnnotateOp", [("operand", "TensorRef"), ("result", "TensorRef"), ("annotation", "string")])
S.table("BreakpointOp", [("operand", "TensorRef")])
S.table("PrintOp", [("operand", "TensorRef"), ("message", "string")])
S.table("MemorySnapshotOp", [("operand", "TensorRef"), ("file_path", "string")])
S.table("RegionStartOp", [("operand", "TensorRef"), ("result", "TensorRef"), ("region_id", "string")])
S.table("RegionEndOp", [("operand", "TensorRef"), ("result", "TensorRef"), ("region_id", "string")])
S.table("PrepareConvTranspose2dWeightsOp", [
    ("weight_tensor", "TensorRef"), ("out", "TensorRef"), ("input_memory_config", "MemoryConfig"),
    ("input_tensor_layout", "TensorLayout"), ("weights_format", "string"), ("in_channels", "u32"),
    ("out_channels", "u32"), ("batch_size", "u32"), ("input_height", "u32"), ("input_width", "u32"),
    ("kernel_size", "[i32]"), ("stride", "[i32]"), ("padding", "[i32]"), ("output_padding", "[i32]"),
    ("dilation", "[i32]"), ("has_bias", "bool"), ("groups", "u32"), ("device", "DeviceRef"),
    ("input_dtype", "DataType"), ("output_dtype", "DataType", OPT), ("conv2d_config", "opaque"),
    ("compute_config", "DeviceComputeKernelConfig"), ("conv2d_slice_config", "opaque"), ("mirror_kernel", "bool", True)])
S.table("PrepareConvTranspose2dBiasOp", [
    ("bias_tensor", "TensorRef"), ("out", "TensorRef"), ("input_memory_config", "MemoryConfig"),
    ("input_tensor_layout", "TensorLayout"), ("in_channels", "u32"), ("out_channels", "u32"), ("batch_size", "u32"),
    ("input_height", "u32"), ("input_width", "u32"), ("kernel_size", "[i32]"), ("stride", "[i32]"),
    ("padding", "[i32]"), ("dilation", "[i32]"), ("groups", "u32"), ("device", "DeviceRef"),
    ("input_dtype", "DataType"), ("output_dtype", "DataType", OPT), ("conv2d_config", "opaque"),
    ("compute_config", "DeviceComputeKernelConfig"), ("conv2d_slice_config", "opaque")])
S.table("NLPCreateQKVHeadsDecodeOp", [
    ("input", "TensorRef"), ("q_out", "TensorRef"), ("k_out", "TensorRef"), ("v_out", "TensorRef"),
    ("num_heads", "u32"), ("num_kv_heads", "u32", OPT), ("overlap_qk_coregrid", "bool", OPT),
    ("batch_offset", "TensorRef"), ("slice_size", "u32", OPT), ("memcfg", "MemoryConfig")])
S.table("NLPConcatHeadsDecodeOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("num_heads", "u32"), ("memcfg", "MemoryConfig")])
S.table("RotaryEmbeddingLlamaOp", [
    ("input", "TensorRef"), ("cos_cache", "TensorRef"), ("sin_cache", "TensorRef"), ("trans_mat", "TensorRef"),
    ("is_decode_mode", "bool"), ("out", "TensorRef"), ("memcfg", "MemoryConfig"),
    ("compute_config", "DeviceComputeKernelConfig")])
S.table("MaxPool2dWithIndicesOp", [
    ("in", "TensorRef"), ("result", "TensorRef"), ("result_indices", "TensorRef"), ("batch_size", "u32"),
    ("input_height", "u32"), ("input_width", "u32"), ("channels", "u32"), ("kernel_size", "[i32]"),
    ("stride", "[i32]"), ("padding", "[i32]"), ("dilation", "[i32]"), ("memory_config", "MemoryConfig"),
    ("applied_shard_scheme", "TensorMemoryLayout", OPT), ("ceil_mode", "bool"),
    ("reallocate_halo_output", "bool", True), ("config_tensors_in_dram", "bool")])
S.table("DropoutOp", [
    ("in", "TensorRef"), ("prob", "f32"), ("scale", "f32"), ("seed", "u32"), ("use_per_device_seed", "bool", True),
    ("output_dtype", "DataType", OPT), ("memory_config", "MemoryConfig"), ("out", "TensorRef")])
S.table("RandOp", [
    ("device", "DeviceRef"), ("size", "[i64]"), ("low", "f32"), ("high", "f32"), ("seed", "u32"),
    ("dtype", "DataType"), ("layout", "TensorLayout"), ("memcfg", "MemoryConfig"), ("out", "TensorRef")])
S.table("BatchNormTrainingOp", [
    ("input", "TensorRef"), ("running_mean", "TensorRef"), ("running_var", "TensorRef"), ("epsilon", "f32"),
    ("momentum", "f32"), ("weight", "TensorRef"), ("bias", "TensorRef"), ("memory_config", "MemoryConfig"),
    ("out", "TensorRef"), ("compute_config", "DeviceComputeKernelConfig")])
S.table("DitRMSNormUnaryFusedOp", [
    ("input", "TensorRef"), ("weight", "TensorRef"), ("bias", "TensorRef"), ("residual_input", "TensorRef"),
    ("epsilon", "f32"), ("activation", "string"), ("memory_config", "MemoryConfig"),
    ("compute_config", "DeviceComputeKernelConfig"), ("out", "TensorRef")])
S.table("DistributedRMSNormOp", [
    ("input", "TensorRef"), ("weight", "TensorRef"), ("residual", "TensorRef"), ("cluster_axis", "u32"), ("epsilon", "f32"),
    ("sub_device_id", "u8", OPT), ("memory_config", "MemoryConfig"), ("num_links", "u32", OPT), ("topology", "Topology", OPT),
    ("compute_config", "DeviceComputeKernelConfig"), ("stats", "TensorRef"), ("program_config", "opaque"),
    ("out", "TensorRef"), ("semaphore", "GlobalSemaphoreRef")])
S.table("RMSNormPreAllGatherOp", [
    ("input", "TensorRef"), ("dtype", "DataType"), ("residual", "TensorRef"), ("memory_config", "MemoryConfig"),
    ("compute_config", "DeviceComputeKernelConfig"), ("program_config", "opaque"), ("use_2d_core_grid", "bool"),
    ("out", "TensorRef")])
S.table("LayerNormPreAllGatherOp", [
    ("input", "TensorRef"), ("residual_input", "TensorRef"), ("recip", "TensorRef"), ("dtype", "DataType", "BFloat16"),
    ("memory_config", "MemoryConfig"), ("compute_config", "DeviceComputeKernelConfig"), ("program_config", "opaque"),
    ("out", "TensorRef")])
S.table("LayerNormPostAllGatherOp", [
    ("input", "TensorRef"), ("stats", "TensorRef"), ("weight", "TensorRef"), ("bias", "TensorRef"), ("epsilon", "f32", 1e-12),
    ("dtype", "DataType", OPT), ("memory_config", "MemoryConfig"), ("compute_config", "DeviceComputeKernelConfig"),
    ("program_config", "opaque"), ("out", "TensorRef")])
S.table("CreateGlobalSemaphoreOp", [("core_range_set", "opaque"), ("initial_value", "u32", OPT), ("out", "GlobalSemaphoreRef")])
S.table("ResetGlobalSemaphoreOp", [("semaphore", "GlobalSemaphoreRef"), ("value", "u32")])
S.table("AllocateMoeComputeSemaphoreOp", [
    ("core_range_set", "opaque"), ("output_height_shard_dim", "u32"), ("hidden_size", "u32"), ("initial_value", "u32", OPT),
    ("out", "GlobalSemaphoreRef")])
S.table("Conv3dOp", [
    ("input", "TensorRef"), ("weight", "TensorRef"), ("bias", "TensorRef"), ("out", "TensorRef"), ("device", "DeviceRef"),
    ("in_channels", "u32"), ("out_channels", "u32"), ("batch_size", "u32"), ("input_depth", "u32"), ("input_height", "u32"),
    ("input_width", "u32"), ("kernel_size", "[i32]"), ("stride", "[i32]"), ("padding", "[i32]"), ("padding_mode", "string"),
    ("groups", "u32"), ("output_dtype", "DataType", OPT), ("conv3d_config", "opaque"),
    ("compute_config", "DeviceComputeKernelConfig"), ("memory_config", "MemoryConfig")])
S.table("PrepareConv3dWeightsOp", [
    ("weight_tensor", "TensorRef"), ("out", "TensorRef"), ("groups", "u32"), ("c_in_block", "u32"), ("alignment", "u32"),
    ("device", "DeviceRef")])
S.enum("ExperimentalEltwiseBinaryBackwardOpType", "u32", ["GeluBW"])
S.table("ExperimentalEltwiseBinaryBackwardOp", [
    ("type", "ExperimentalEltwiseBinaryBackwardOpType"), ("grad", "TensorRef"), ("input", "TensorRef"), ("approximate", "string"),
    ("output_dtype", "DataType", OPT), ("memory_config", "MemoryConfig"), ("out", "TensorRef")])
S.table("EmbeddingBackwardOp", [
    ("input", "TensorRef"), ("weight", "TensorRef"), ("in_grad", "TensorRef"), ("dtype", "DataType", OPT), ("memcfg", "MemoryConfig"),
    ("out", "TensorRef")])
S.table("AdamWOp", [
    ("param", "TensorRef"), ("grad", "TensorRef"), ("exp_avg", "TensorRef"), ("exp_avg_sq", "TensorRef"),
    ("max_exp_avg_sq", "TensorRef"), ("lr", "f32"), ("beta1", "f32"), ("beta2", "f32"), ("beta1_pow", "f32"), ("beta2_pow", "f32"),
    ("epsilon", "f32"), ("weight_decay", "f32"), ("stochastic_rounding", "bool")])
S.table("ChunkedScaledDotProductAttentionOp", [
    ("query", "TensorRef"), ("key", "TensorRef"), ("value", "TensorRef"), ("page_table", "TensorRef"),
    ("chunk_start_idx", "TensorRef"), ("scale", "f32", OPT), ("out", "TensorRef"), ("memcfg", "MemoryConfig"),
    ("program_config", "opaque")])
S.table("FlashMlaPrefillOp", [
    ("query", "TensorRef"), ("key", "TensorRef"), ("value", "TensorRef"), ("attention_mask", "TensorRef"),
    ("head_dim_v", "u32"), ("is_causal", "bool"), ("scale", "f32", OPT), ("out", "TensorRef"), ("memcfg", "MemoryConfig")])
S.table("IndexerScoreDsaOp", [
    ("query", "TensorRef"), ("key", "TensorRef"), ("weights", "TensorRef"), ("chunk_start_idx", "u32"), ("out", "TensorRef"),
    ("cluster_axis", "u32", OPT)])
S.table("PagedFlashMultiLatentAttentionDecodeOp", [
    ("query", "TensorRef"), ("key", "TensorRef"), ("value", "TensorRef"), ("head_dim_v", "u32"), ("page_table", "TensorRef"),
    ("is_causal", "bool"), ("attention_mask", "TensorRef"), ("cur_pos_tensor", "TensorRef"), ("attention_sink", "TensorRef"),
    ("scale", "f32", OPT), ("out", "TensorRef"), ("memcfg", "MemoryConfig")])
S.table("UniformScale2D", [("scale", "i32")])
S.table("NonUniformScale2D", [("scale", "[i32]")])
S.union("Scale2D", ["UniformScale2D", "NonUniformScale2D"])
S.table("UpsampleOp", [
    ("in", "TensorRef"), ("scale_factor", "Scale2D"), ("mode", "string"), ("memory_config", "MemoryConfig"),
    ("out", "TensorRef")])
S.table("PrepareConv2dWeightsOp", [
    ("weight_tensor", "TensorRef"), ("out", "TensorRef"), ("input_memory_config", "MemoryConfig"),
    ("input_tensor_layout", "TensorLayout"), ("weights_format", "string"), ("in_channels", "u32"),
    ("out_channels", "u32"), ("batch_size", "u32"), ("input_height", "u32"), ("input_width", "u32"),
    ("kernel_size", "[i32]"), ("stride", "[i32]"), ("padding", "[i32]"), ("dilation", "[i32]"), ("has_bias", "bool"),
    ("groups", "u32"), ("device", "DeviceRef"), ("input_dtype", "DataType"), ("output_dtype", "DataType", OPT),
    ("conv2d_config", "opaque"), ("compute_config", "DeviceComputeKernelConfig"), ("conv2d_slice_config", "opaque")])
S.table("PrepareConv2dBiasOp", [
    ("bias_tensor", "TensorRef"), ("out", "TensorRef"), ("input_memory_config", "MemoryConfig"),
    ("input_tensor_layout", "TensorLayout"), ("in_channels", "u32"), ("out_channels", "u32"), ("batch_size", "u32"),
    ("input_height", "u32"), ("input_width", "u32"), ("kernel_size", "[i32]"), ("stride", "[i32]"), ("padding", "[i32]"),
    ("dilation", "[i32]"), ("groups", "u32"), ("device", "DeviceRef"), ("input_dtype", "DataType"),
    ("output_dtype", "DataType", OPT), ("conv2d_config", "opaque"), ("compute_config", "DeviceComputeKernelConfig"),
    ("conv2d_slice_config", "opaque")])
# operations/data_movement.fbs: gather / scatter / sort; operations/reduction.fbs: top-k / sampling
S.enum("ScatterReduceType", "u8", {"Sum": 0, "Max": 2, "Min": 3, "Prod": 6, "Invalid": 7})
S.table("ScatterOp", [
    ("input", "TensorRef"), ("out", "TensorRef"), ("index", "TensorRef"), ("source", "TensorRef"), ("dim", "i32"),
    ("memory_config", "MemoryConfig"), ("scatter_reduce_type", "ScatterReduceType")])
S.table("GatherOp", [
    ("input", "TensorRef"), ("index", "TensorRef"), ("out", "TensorRef"), ("dim", "i32"), ("memory_config", "MemoryConfig")])
S.table("SortOp", [
    ("in", "TensorRef"), ("dim", "i8"), ("descending", "bool"), ("stable", "bool"), ("memcfg", "MemoryConfig"),
    ("outputs", "[TensorRef]")])
S.table("TopKOp", [
    ("input_tensor", "TensorRef"), ("k", "i32"), ("dim", "i32", -1), ("largest", "bool", True), ("sorted", "bool", True),
    ("memcfg", "MemoryConfig"), ("outputs", "[TensorRef]")])
S.table("SamplingOp", [
    ("input_values", "TensorRef"), ("input_indices", "TensorRef"), ("k", "TensorRef"), ("p", "TensorRef"), ("temp", "TensorRef"),
    ("seed", "u32", OPT), ("out", "TensorRef")])
# operations/embedding.fbs
S.table("EmbeddingOp", [("input", "TensorRef"), ("weight", "TensorRef"), ("out", "TensorRef")])
# operations/pool.fbs
S.enum("Pool2dOpType", "u32", ["AvgPool2d", "MaxPool2d"])
S.table("AvgPool2dExtraParams", [("count_include_pad", "bool")])
S.table("MaxPool2dExtraParams", [])
S.union("Pool2dExtraParams", ["AvgPool2dExtraParams", "MaxPool2dExtraParams"])
S.table("Pool2dOp", [
    ("type", "Pool2dOpType"), ("in", "TensorRef"), ("out", "TensorRef"), ("batch_size", "u32"),
    ("input_height", "u32"), ("input_width", "u32"), ("channels", "u32"), ("kernel_size", "[i32]"),
    ("stride", "[i32]"), ("padding", "[i32]"), ("dilation", "[i32]"), ("extra_params", "Pool2dExtraParams"),
    ("memory_config", "MemoryConfig"), ("applied_shard_scheme", "TensorMemoryLayout", OPT),
    ("ceil_mode", "bool"), ("reallocate_halo_output", "bool", True), ("config_tensors_in_dram", "bool")])
S.table("GlobalAvgPool2dOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("memory_config", "MemoryConfig"), ("dtype", "DataType", OPT)])

# --- data movement (operations/data_movement.fbs)
S.table("ConcatOp", [
    ("inputs", "[TensorRef]"), ("out", "TensorRef"), ("dim", "i32"),
    ("memory_config", "MemoryConfig")])
S.table("PermuteOp", [
    ("in", "TensorRef"), ("permutation", "[i64]"), ("memory_config", "MemoryConfig"),
    ("pad_value", "f32"), ("out", "TensorRef")])
S.table("RepeatInterleaveOp", [
    ("input", "TensorRef"), ("out", "TensorRef"), ("repeats", "u32"), ("dim", "i32"),
    ("memory_config", "MemoryConfig")])
S.table("RepeatOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("repeat_dims", "[i64]"), ("memcfg", "MemoryConfig")])
S.table("ReshapeOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("shape", "[i32]"), ("memory_config", "MemoryConfig")])
S.enum("SliceOpType", "u32", ["SliceStaticOp", "SliceDynamicOp"])
S.table("SliceStaticOpParams", [("begins", "[i64]"), ("ends", "[i64]")])
S.table("SliceDynamicOpParams", [("begins", "TensorRef"), ("ends", "TensorRef")])
S.union("SliceOpParams", ["SliceStaticOpParams", "SliceDynamicOpParams"])
S.table("SliceOp", [
    ("type", "SliceOpType"), ("in", "TensorRef"), ("out", "TensorRef"), ("step", "[i64]"),
    ("params", "SliceOpParams")])
S.table("TransposeOp", [("in", "TensorRef"), ("out", "TensorRef"), ("dim0", "i32"), ("dim1", "i32")])
S.table("PadOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("padding", "[u32]"), ("value", "f32"),
    ("use_multicore", "bool"), ("memcfg", "MemoryConfig")])

# --- transformer (operations/transformer.fbs)
S.table("ConcatenateHeadsOp", [("in", "TensorRef"), ("out", "TensorRef"), ("memcfg", "MemoryConfig")])
S.table("RotaryEmbeddingOp", [
    ("input", "TensorRef"), ("cos_cache", "TensorRef"), ("sin_cache", "TensorRef"),
    ("token_index", "u32", OPT), ("out", "TensorRef"), ("memcfg", "MemoryConfig"),
    ("compute_config", "DeviceComputeKernelConfig")])
S.table("ScaledDotProductAttentionOp", [
    ("query", "TensorRef"), ("key", "TensorRef"), ("value", "TensorRef"), ("is_causal", "bool"),
    ("attention_mask", "TensorRef"), ("scale", "f32", OPT), ("sliding_window_size", "u32", OPT),
    ("attention_sink", "TensorRef"), ("out", "TensorRef"), ("memcfg", "MemoryConfig")])
S.table("SplitQueryKeyValueAndSplitHeadsOp", [
    ("in", "TensorRef"), ("kv_input", "TensorRef"), ("q_out", "TensorRef"), ("k_out", "TensorRef"),
    ("v_out", "TensorRef"), ("num_heads", "u32"), ("num_kv_heads", "u32", OPT),
    ("transpose_key", "bool"), ("memcfg", "MemoryConfig")])

S.table("ScaledDotProductAttentionDecodeOp", [
    ("query", "TensorRef"), ("key", "TensorRef"), ("value", "TensorRef"), ("is_causal", "bool"),
    ("attention_mask", "TensorRef"), ("cur_pos_tensor", "TensorRef"), ("attention_sink", "TensorRef"),
    ("scale", "f32", OPT), ("sliding_window_size", "u32", OPT), ("out", "TensorRef"),
    ("memcfg", "MemoryConfig"), ("program_config", "opaque")])
# operations/kv_cache.fbs
S.table("FillCacheOp", [("cache", "TensorRef"), ("input", "TensorRef"), ("batch_offset", "u32")])
S.table("UpdateCacheOp", [
    ("cache", "TensorRef"), ("input", "TensorRef"), ("update_index", "TensorRef"), ("batch_offset", "u32")])
S.table("PagedUpdateCacheOp", [
    ("cache", "TensorRef"), ("input", "TensorRef"), ("update_index", "TensorRef"), ("share_cache", "bool"),
    ("page_table", "TensorRef")])
S.table("PagedFillCacheOp", [
    ("cache", "TensorRef"), ("input", "TensorRef"), ("page_table", "TensorRef"), ("batch_idx_tensor", "TensorRef")])
# operations/transformer.fbs
S.table("PagedScaledDotProductAttentionDecodeOp", [
    ("query", "TensorRef"), ("key", "TensorRef"), ("value", "TensorRef"), ("page_table", "TensorRef"), ("is_causal", "bool"),
    ("attention_mask", "TensorRef"), ("cur_pos_tensor", "TensorRef"), ("attention_sink", "TensorRef"),
    ("scale", "f32", OPT), ("sliding_window_size", "u32", OPT), ("out", "TensorRef"), ("memcfg", "MemoryConfig"),
    ("program_config", "opaque")])

# --- ccl (operations/ccl.fbs)
S.table("AllGatherOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("all_gather_dim", "i32"), ("cluster_axis", "u32"),
    ("sub_device_id", "u8", OPT), ("memory_config", "MemoryConfig"), ("num_links", "u32", OPT),
    ("topology", "Topology", OPT)])
S.table("AllReduceOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("reduce_type", "u32"), ("cluster_axis", "u32"),
    ("sub_device_id", "u8", OPT), ("memory_config", "MemoryConfig"), ("num_links", "u32", OPT),
    ("topology", "Topology", OPT)])
S.table("AllReduceAsyncOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("reduce_type", "u32"), ("cluster_axis", "u32"),
    ("sub_device_id", "u8", OPT), ("memory_config", "MemoryConfig"), ("num_links", "u32", OPT),
    ("topology", "Topology", OPT)])
S.table("PointToPointOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("sender_coord", "[u32]"), ("receiver_coord", "[u32]"),
    ("optional_output_tensor", "TensorRef")])
S.table("AllToAllDispatchOp", [
    ("input_tensor", "TensorRef"), ("expert_indices", "TensorRef"), ("expert_mapping", "TensorRef"),
    ("dispatched", "TensorRef"), ("metadata", "TensorRef"), ("num_devices", "u32"), ("cluster_axis", "u32"),
    ("memory_config", "MemoryConfig")])
S.table("AllToAllCombineOp", [
    ("input_tensor", "TensorRef"), ("expert_metadata", "TensorRef"), ("expert_mapping", "TensorRef"), ("out", "TensorRef"),
    ("num_devices", "u32"), ("cluster_axis", "u32"), ("num_experts_per_tok", "u32"), ("output_shard_dim", "u32", 2),
    ("memory_config", "MemoryConfig")])
S.table("MoeExpertTokenRemapOp", [
    ("topk_tensor", "TensorRef"), ("expert_mapping", "TensorRef"), ("expert_metadata", "TensorRef"), ("mapping", "TensorRef"),
    ("reduced", "TensorRef"), ("reduction_size", "u32"), ("memory_config", "MemoryConfig")])
S.table("SparseMatmulOp", [
    ("a", "TensorRef"), ("b", "TensorRef"), ("sparsity", "TensorRef"), ("out", "TensorRef"), ("is_input_a_sparse", "bool"),
    ("is_input_b_sparse", "bool"), ("nnz", "i64", OPT), ("program_config", "opaque"), ("memory_config", "MemoryConfig"),
    ("dtype", "DataType"), ("compute_config", "DeviceComputeKernelConfig")])
S.table("AllToAllDispatchMetadataOp", [
    ("input_tensor", "TensorRef"), ("expert_indices", "TensorRef"), ("expert_scores", "TensorRef"),
    ("expert_mapping", "TensorRef"), ("dispatched", "TensorRef"), ("indices", "TensorRef"), ("scores", "TensorRef"),
    ("num_devices", "u32"), ("cluster_axis", "u32"), ("memory_config", "MemoryConfig"),
    ("dispatched_buffer", "TensorRef"), ("indices_buffer", "TensorRef"), ("scores_buffer", "TensorRef"),
    ("cross_device_semaphore", "GlobalSemaphoreRef")])
S.table("TopKRouterGptOp", [
    ("input", "TensorRef"), ("weight", "TensorRef"), ("bias", "TensorRef"), ("k", "i32"), ("num_experts", "i32"),
    ("expert_indices", "TensorRef"), ("expert_weights", "TensorRef")])
S.table("ReduceScatterOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("scatter_dim", "i32"), ("reduce_type", "u32"),
    ("cluster_axis", "u32"), ("sub_device_id", "u8", OPT), ("memory_config", "MemoryConfig"),
    ("num_links", "u32", OPT), ("topology", "Topology", OPT),
    ("compute_config", "DeviceComputeKernelConfig")])
S.table("DistributeTensorOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("mapper_config", "MeshMapperConfig"),
    ("device", "DeviceRef"), ("cq_id", "u32", OPT)])
S.table("AggregateTensorOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("composer_config", "MeshComposerConfig"),
    ("device", "DeviceRef")])
S.table("MeshPartitionOp", [
    ("in", "TensorRef"), ("out", "TensorRef"), ("dim", "i32"), ("cluster_axis", "u32", OPT),
    ("memory_config", "MemoryConfig")])

# --- sub-programs: const-eval cache, calls, traces (operations/load_cached.fbs, mlir_native.fbs,
#     trace.fbs) and the two copies the trace functions use (operations/data_movement.fbs)
S.table("LoadCachedOp", [
    ("inputs", "[TensorRef]"), ("callee_name", "string"), ("program_idx", "u32"),
    ("outputs", "[TensorRef]"), ("program_hash", "string")])
S.table("FuncCallOp", [
    ("program_id", "u32"), ("inputs", "[TensorRef]"), ("outputs", "[TensorRef]"),
    ("semaphore_inputs", "[GlobalSemaphoreRef]")])
S.table("BeginTraceCaptureOp", [("device", "DeviceRef"), ("trace_id", "TensorRef"), ("cq_id", "u32")])
S.table("EndTraceCaptureOp", [("device", "DeviceRef"), ("trace_id", "TensorRef"), ("cq_id", "u32")])
S.table("ExecuteTraceOp", [
    ("device", "DeviceRef"), ("trace_id", "TensorRef"), ("cq_id", "u32"), ("blocking", "bool")])
S.table("CaptureOrExecuteTraceOp", [
    ("device", "DeviceRef"), ("capture_program_id", "u32"), ("execute_program_id", "u32"),
    ("allocate_slots_program_id", "u32"), ("inputs", "[TensorRef]"), ("outputs", "[TensorRef]"),
    ("semaphore_inputs", "[GlobalSemaphoreRef]")])
S.table("WriteTensorOp", [
    ("host_tensor", "TensorRef"), ("device_tensor", "TensorRef"), ("blocking", "bool"), ("cq_id", "u32")])
S.table("CopyOp", [("src", "TensorRef"), ("dst", "TensorRef")])

# --- program (TTNN/program.fbs).  Union member order fixes the op type ids.
OP_TYPE_MEMBERS = [
    "AdamWOp", "AggregateTensorOp", "AllGatherOp", "AllReduceAsyncOp", "AllReduceOp",
    "AllToAllCombineOp", "AllToAllDispatchMetadataOp", "AllToAllDispatchOp", "ArangeOp",
    "AssignOp", "BatchNormInferenceOp", "BatchNormTrainingOp", "BitcastConvertOp",
    "BeginTraceCaptureOp", "CaptureOrExecuteTraceOp", "ChunkedScaledDotProductAttentionOp",
    "ConcatOp", "ConcatenateHeadsOp", "RotaryEmbeddingLlamaOp", "RotaryEmbeddingOp",
    "NLPCreateQKVHeadsDecodeOp", "NLPConcatHeadsOp", "ConstantOp", "Conv1dOp", "Conv2dOp",
    "ConvTranspose2dOp", "Conv3dOp", "CpuOp", "DeallocateOp", "DistributeTensorOp",
    "DistributedRMSNormOp", "DitRMSNormUnaryFusedOp", "DropoutOp", "EltwiseBinaryCompositeOp",
    "EltwiseBinaryCompositeScalarOp", "EltwiseBinaryOp", "EltwiseQuantizationOp",
    "EltwiseTernaryWhereOp", "EltwiseUnaryCompositeOp", "EltwiseUnaryOp", "EmbeddingBackwardOp",
    "EmbeddingOp", "EmptyOp", "EndTraceCaptureOp", "ExecuteTraceOp",
    "ExperimentalEltwiseBinaryBackwardOp", "FillCacheOp", "FromDeviceOp", "FullOp", "FuncCallOp",
    "GatherOp", "GenericOp", "GetDeviceOp", "GlobalAvgPool2dOp", "GroupNormOp",
    "IndexerScoreDsaOp", "LayerNormOp", "LayerNormPreAllGatherOp", "LayerNormPostAllGatherOp",
    "LinearOp", "LoadCachedOp", "MatmulOp", "SparseMatmulOp", "MaxPool2dWithIndicesOp",
    "MeshPartitionOp", "MoeExpertTokenRemapOp", "MoeGptOp", "PrepareMoEComputeW0W1WeightsOp",
    "PrepareMoEComputeW2WeightsOp", "MoeComputeOp", "CumSumOp", "CumProdOp", "NamedFullOp",
    "NLPConcatHeadsDecodeOp", "PadOp", "PagedFillCacheOp",
    "PagedFlashMultiLatentAttentionDecodeOp", "PagedScaledDotProductAttentionDecodeOp",
    "PagedUpdateCacheOp", "PermuteOp", "PointToPointOp", "Pool2dOp", "PrepareConv2dBiasOp",
    "PrepareConv2dWeightsOp", "PrepareConv3dWeightsOp", "PrepareConvTranspose2dBiasOp",
    "PrepareConvTranspose2dWeightsOp", "RandOp", "ReductionArgMaxOp", "ReductionOp",
    "ReductionProdOp", "ReduceScatterOp", "RepeatInterleaveOp", "RepeatOp",
    "RMSNormPreAllGatherOp", "RMSNormOp", "ReshapeOp", "SamplingOp",
    "ScaledDotProductAttentionOp", "ScaledDotProductAttentionDecodeOp", "FlashMlaPrefillOp",
    "ScatterOp", "SDPAForwardOp", "SDPABackwardOp", "SelectiveReduceCombineOp", "SliceOp",
    "SoftmaxOp", "SortOp", "SplitQueryKeyValueAndSplitHeadsOp", "ToDeviceOp", "ToLayoutOp",
    "ToMemoryConfigOp", "TransposeOp", "TypecastOp", "UpdateCacheOp", "UpsampleOp",
    "WriteTensorOp", "DumpTensorOp", "LoadTensorOp", "AnnotateOp", "BreakpointOp", "PrintOp",
    "MemorySnapshotOp", "RegionStartOp", "RegionEndOp", "TopKOp", "TopKRouterGptOp",
    "CreateGlobalSemaphoreOp", "ResetGlobalSemaphoreOp", "AllocateMoeComputeSemaphoreOp",
    "CopyOp",
]
# Members without a declared table stay in the union as names only.
for _m in OP_TYPE_MEMBERS:
    if _m not in S.tables:
        S.table(_m, [])
UNDECLARED_OPS = [m for m in OP_TYPE_MEMBERS if not S.tables[m].fields]
S.union("OpType", OP_TYPE_MEMBERS)

S.table("Operation", [("type", "OpType"), ("debug_info", "string"), ("loc_info", "string")])
S.table("Program", [
    ("name", "string"), ("inputs", "[TensorRef]"), ("outputs", "[TensorRef]"),
    ("operations", "[Operation]"), ("dylibs", "[DynamicLib]"), ("debug_info", "DebugInfo"),
    ("private", "bool"), ("mesh_shape", "Dim2d"), ("semaphore_inputs", "[GlobalSemaphoreRef]")])
S.table("TTNNBinary", [
    ("version", "Version"), ("schema_hash", "string"), ("ttmlir_git_hash", "string"),
    ("system_desc", "SystemDesc"), ("mlir", "MLIR"), ("programs", "[Program]")])

FILE_IDENTIFIER = b"TTNN"
# flatc hashes its .bfbs output to get the schema hash (cmake/modules/BuildFlatbuffers.cmake);
# that cannot be reproduced without flatc, so this runtime uses its own constant.
SCHEMA_HASH = "b200-ttnn-schema-v1"
