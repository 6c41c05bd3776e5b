// Program executor: runs one program of a TTNN binary on a (mesh) device.
//
// Counterpart of ProgramExecutor / ProgramTensorPool in the reference
// (runtime/lib/ttnn/program_executor.cpp:146-266,285-755; runtime/lib/ttnn/types/types.cpp:108-232)
// with the per-op adapters of runtime/lib/ttnn/operations/** folded in.  Differences that
// come from the target:
//   * every op ends in a launch on a CUDA stream (one stream per mesh coordinate) instead of a
//     call into tt-metal; nothing synchronises until the caller reads a result;
//   * a peephole pass over the op list fuses chains the flatbuffer spells as separate ops
//     (quantize->requantize->dequantize, matmul->add->activation, silu*mul, add->rms_norm,
//     dequantize(weight)->linear) into single launches.  A fused launch keeps the rounding
//     points of the chain it replaces, so results equal the op-by-op execution bit for bit.
//     Fusion is off while debug hooks are registered, because callbacks may ask for any
//     intermediate tensor;
//   * tilize / untilize and memory-config changes are metadata only.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <map>
#include <unordered_map>
#include <unordered_set>

#include "impl.h"
#include "tt/runtime/debug.h"
#include "tt/runtime/perf.h"
#include "tt/runtime/runtime.h"

namespace tt::runtime::cuda {

namespace fbt = ::tt::target::ttnn;
using fbt::OpType;
using ::tt::target::TensorLayout;

// ---- static facts about a program, computed once per (binary, program) -----------------------
struct ProgramInfo {
  std::unordered_map<uint32_t, uint32_t> useCount; // consumers other than DeallocateOp
  std::unordered_map<uint32_t, uint32_t> firstUse; // index of the first such consumer
  std::unordered_set<uint32_t> outputs;
  // CopyOp(src -> dst): when the copy is src's only use and dst's only use, src's producer writes
  // into dst's memory and the copy has nothing left to do.
  std::unordered_map<uint32_t, const fbt::TensorRef *> copyTarget;
};

static void pushRef(std::vector<const fbt::TensorRef *> &v, const fbt::TensorRef *r) {
  if (r) v.push_back(r);
}

static void quantParamRefs(const fbt::EltwiseQuantizationOp *op, std::vector<const fbt::TensorRef *> &ins) {
  auto scaleRef = [&](fbt::QuantizationScale ty, const void *p) {
    if (ty == fbt::QuantizationScale::PerAxisScale && p) pushRef(ins, static_cast<const fbt::PerAxisScale *>(p)->scale());
  };
  auto zpRef = [&](fbt::QuantizationZeroPoint ty, const void *p) {
    if (ty == fbt::QuantizationZeroPoint::PerAxisZeroPoint && p)
      pushRef(ins, static_cast<const fbt::PerAxisZeroPoint *>(p)->zero_point());
  };
  if (const auto *qd = op->params_as_QuantizeDequantizeOpParams()) {
    scaleRef(qd->scale_type(), qd->scale());
    zpRef(qd->zero_point_type(), qd->zero_point());
  } else if (const auto *rq = op->params_as_RequantizeOpParams()) {
    scaleRef(rq->in_scale_type(), rq->in_scale());
    zpRef(rq->in_zero_point_type(), rq->in_zero_point());
    scaleRef(rq->out_scale_type(), rq->out_scale());
    zpRef(rq->out_zero_point_type(), rq->out_zero_point());
  }
}

void collectOpRefs(const fbt::Operation *op, std::vector<const fbt::TensorRef *> &ins,
                   std::vector<const fbt::TensorRef *> &outs) {
  switch (op->type_type()) {
#define IN1_OUT(T, inName)                                                               \
  case OpType::T: {                                                                      \
    const auto *o = op->type_as_##T();                                                   \
    pushRef(ins, o->inName());                                                           \
    pushRef(outs, o->out());                                                             \
    break;                                                                               \
  }
    IN1_OUT(EltwiseUnaryOp, in)
    IN1_OUT(EltwiseUnaryCompositeOp, in)
    IN1_OUT(FromDeviceOp, in)
    IN1_OUT(ToDeviceOp, in)
    IN1_OUT(ToLayoutOp, in)
    IN1_OUT(ToMemoryConfigOp, in0)
    IN1_OUT(TypecastOp, in)
    IN1_OUT(ReductionOp, in)
    IN1_OUT(SoftmaxOp, in)
    IN1_OUT(PermuteOp, in)
    IN1_OUT(RepeatInterleaveOp, input)
    IN1_OUT(RepeatOp, in)
    IN1_OUT(ReshapeOp, in)
    IN1_OUT(SliceOp, in)
    IN1_OUT(TransposeOp, in)
    IN1_OUT(ConcatenateHeadsOp, in)
    IN1_OUT(AllGatherOp, in)
    IN1_OUT(AllReduceOp, in)
    IN1_OUT(ReduceScatterOp, in)
    IN1_OUT(DistributeTensorOp, in)
    IN1_OUT(AggregateTensorOp, in)
    IN1_OUT(MeshPartitionOp, in)
    IN1_OUT(ReductionArgMaxOp, in)
    IN1_OUT(CumSumOp, in)
    IN1_OUT(CumProdOp, in)
    IN1_OUT(BitcastConvertOp, in)
    IN1_OUT(NLPConcatHeadsOp, in)
    IN1_OUT(ReductionProdOp, in)
    IN1_OUT(UpsampleOp, in)
    IN1_OUT(PrepareConv2dWeightsOp, weight_tensor)
    IN1_OUT(PrepareConv2dBiasOp, bias_tensor)
    IN1_OUT(Pool2dOp, in)
    IN1_OUT(GlobalAvgPool2dOp, in)
    IN1_OUT(PadOp, in)
#undef IN1_OUT
  case OpType::AllToAllDispatchOp: {
    const auto *o = op->type_as_AllToAllDispatchOp();
    pushRef(ins, o->input_tensor());
    pushRef(ins, o->expert_indices());
    pushRef(ins, o->expert_mapping());
    pushRef(outs, o->dispatched());
    pushRef(outs, o->metadata());
    break;
  }
  case OpType::PagedFlashMultiLatentAttentionDecodeOp: {
    const auto *o = op->type_as_PagedFlashMultiLatentAttentionDecodeOp();
    pushRef(ins, o->query());
    pushRef(ins, o->key());
    pushRef(ins, o->value());
    pushRef(ins, o->page_table());
    pushRef(ins, o->attention_mask());
    pushRef(ins, o->cur_pos_tensor());
    pushRef(ins, o->attention_sink());
    pushRef(outs, o->out());
    break;
  }
  case OpType::IndexerScoreDsaOp: {
    const auto *o = op->type_as_IndexerScoreDsaOp();
    pushRef(ins, o->query());
    pushRef(ins, o->key());
    pushRef(ins, o->weights());
    pushRef(outs, o->out());
    break;
  }
  case OpType::FlashMlaPrefillOp: {
    const auto *o = op->type_as_FlashMlaPrefillOp();
    pushRef(ins, o->query());
    pushRef(ins, o->key());
    pushRef(ins, o->value());
    pushRef(ins, o->attention_mask());
    pushRef(outs, o->out());
    break;
  }
  case OpType::ChunkedScaledDotProductAttentionOp: {
    const auto *o = op->type_as_ChunkedScaledDotProductAttentionOp();
    pushRef(ins, o->query());
    pushRef(ins, o->key());
    pushRef(ins, o->value());
    pushRef(ins, o->page_table());
    pushRef(ins, o->chunk_start_idx());
    pushRef(outs, o->out());
    break;
  }
  case OpType::Conv3dOp: {
    const auto *o = op->type_as_Conv3dOp();
    pushRef(ins, o->input());
    pushRef(ins, o->weight());
    pushRef(ins, o->bias());
    pushRef(outs, o->out());
    break;
  }
  case OpType::PrepareConv3dWeightsOp: {
    const auto *o = op->type_as_PrepareConv3dWeightsOp();
    pushRef(ins, o->weight_tensor());
    pushRef(outs, o->out());
    break;
  }
  case OpType::ExperimentalEltwiseBinaryBackwardOp: {
    const auto *o = op->type_as_ExperimentalEltwiseBinaryBackwardOp();
    pushRef(ins, o->grad());
    pushRef(ins, o->input());
    pushRef(outs, o->out());
    break;
  }
  case OpType::EmbeddingBackwardOp: {
    const auto *o = op->type_as_EmbeddingBackwardOp();
    pushRef(ins, o->input());
    pushRef(ins, o->weight());
    pushRef(ins, o->in_grad());
    pushRef(outs, o->out());
    break;
  }
  case OpType::AdamWOp: {
    const auto *o = op->type_as_AdamWOp();
    pushRef(ins, o->param());
    pushRef(ins, o->grad());
    pushRef(ins, o->exp_avg());
    pushRef(ins, o->exp_avg_sq());
    pushRef(ins, o->max_exp_avg_sq());
    break;
  }
  case OpType::AllToAllDispatchMetadataOp: {
    const auto *o = op->type_as_AllToAllDispatchMetadataOp();
    pushRef(ins, o->input_tensor());
    pushRef(ins, o->expert_indices());
    pushRef(ins, o->expert_scores());
    pushRef(ins, o->expert_mapping());
    pushRef(ins, o->dispatched_buffer());
    pushRef(ins, o->indices_buffer());
    pushRef(ins, o->scores_buffer());
    pushRef(outs, o->dispatched());
    pushRef(outs, o->indices());
    pushRef(outs, o->scores());
    break;
  }
  case OpType::TopKRouterGptOp: {
    const auto *o = op->type_as_TopKRouterGptOp();
    pushRef(ins, o->input());
    pushRef(ins, o->weight());
    pushRef(ins, o->bias());
    pushRef(outs, o->expert_indices());
    pushRef(outs, o->expert_weights());
    break;
  }
  case OpType::AllToAllCombineOp: {
    const auto *o = op->type_as_AllToAllCombineOp();
    pushRef(ins, o->input_tensor());
    pushRef(ins, o->expert_metadata());
    pushRef(ins, o->expert_mapping());
    pushRef(outs, o->out());
    break;
  }
  case OpType::MoeExpertTokenRemapOp: {
    const auto *o = op->type_as_MoeExpertTokenRemapOp();
    pushRef(ins, o->topk_tensor());
    pushRef(ins, o->expert_mapping());
    pushRef(ins, o->expert_metadata());
    pushRef(outs, o->mapping());
    pushRef(outs, o->reduced());
    break;
  }
  case OpType::SparseMatmulOp: {
    const auto *o = op->type_as_SparseMatmulOp();
    pushRef(ins, o->a());
    pushRef(ins, o->b());
    pushRef(ins, o->sparsity());
    pushRef(outs, o->out());
    break;
  }
  case OpType::DitRMSNormUnaryFusedOp: {
    const auto *o = op->type_as_DitRMSNormUnaryFusedOp();
    pushRef(ins, o->input());
    pushRef(ins, o->weight());
    pushRef(ins, o->bias());
    pushRef(ins, o->residual_input());
    pushRef(outs, o->out());
    break;
  }
  case OpType::DistributedRMSNormOp: {
    const auto *o = op->type_as_DistributedRMSNormOp();
    pushRef(ins, o->input());
    pushRef(ins, o->weight());
    pushRef(ins, o->residual());
    pushRef(ins, o->stats());
    pushRef(outs, o->out());
    break;
  }
  case OpType::RMSNormPreAllGatherOp: {
    const auto *o = op->type_as_RMSNormPreAllGatherOp();
    pushRef(ins, o->input());
    pushRef(ins, o->residual());
    pushRef(outs, o->out());
    break;
  }
  case OpType::LayerNormPreAllGatherOp: {
    const auto *o = op->type_as_LayerNormPreAllGatherOp();
    pushRef(ins, o->input());
    pushRef(ins, o->residual_input());
    pushRef(ins, o->recip());
    pushRef(outs, o->out());
    break;
  }
  case OpType::LayerNormPostAllGatherOp: {
    const auto *o = op->type_as_LayerNormPostAllGatherOp();
    pushRef(ins, o->input());
    pushRef(ins, o->stats());
    pushRef(ins, o->weight());
    pushRef(ins, o->bias());
    pushRef(outs, o->out());
    break;
  }
  case OpType::CreateGlobalSemaphoreOp:
  case OpType::ResetGlobalSemaphoreOp:
  case OpType::AllocateMoeComputeSemaphoreOp: break; // no tensors
  case OpType::AssignOp: {
    const auto *o = op->type_as_AssignOp();
    pushRef(ins, o->input());
    pushRef(outs, o->output());
    break;
  }
  case OpType::EltwiseBinaryCompositeScalarOp: {
    const auto *o = op->type_as_EltwiseBinaryCompositeScalarOp();
    pushRef(ins, o->lhs());
    pushRef(outs, o->out());
    break;
  }
  case OpType::DumpTensorOp: pushRef(ins, op->type_as_DumpTensorOp()->in()); break;
  case OpType::LoadTensorOp: pushRef(outs, op->type_as_LoadTensorOp()->out()); break;
  case OpType::AnnotateOp: {
    const auto *o = op->type_as_AnnotateOp();
    pushRef(ins, o->operand());
    pushRef(outs, o->result());
    break;
  }
  case OpType::RegionStartOp: {
    const auto *o = op->type_as_RegionStartOp();
    pushRef(ins, o->operand());
    pushRef(outs, o->result());
    break;
  }
  case OpType::RegionEndOp: {
    const auto *o = op->type_as_RegionEndOp();
    pushRef(ins, o->operand());
    pushRef(outs, o->result());
    break;
  }
  case OpType::BreakpointOp: pushRef(ins, op->type_as_BreakpointOp()->operand()); break;
  case OpType::PrintOp: pushRef(ins, op->type_as_PrintOp()->operand()); break;
  case OpType::MemorySnapshotOp: pushRef(ins, op->type_as_MemorySnapshotOp()->operand()); break;
  case OpType::AllReduceAsyncOp: {
    const auto *o = op->type_as_AllReduceAsyncOp();
    pushRef(ins, o->in());
    pushRef(outs, o->out());
    break;
  }
  case OpType::PointToPointOp: {
    const auto *o = op->type_as_PointToPointOp();
    pushRef(ins, o->in());
    pushRef(ins, o->optional_output_tensor());
    pushRef(outs, o->out());
    break;
  }
  case OpType::PrepareConvTranspose2dWeightsOp: {
    const auto *o = op->type_as_PrepareConvTranspose2dWeightsOp();
    pushRef(ins, o->weight_tensor());
    pushRef(outs, o->out());
    break;
  }
  case OpType::PrepareConvTranspose2dBiasOp: {
    const auto *o = op->type_as_PrepareConvTranspose2dBiasOp();
    pushRef(ins, o->bias_tensor());
    pushRef(outs, o->out());
    break;
  }
  case OpType::NLPCreateQKVHeadsDecodeOp: {
    const auto *o = op->type_as_NLPCreateQKVHeadsDecodeOp();
    pushRef(ins, o->input());
    pushRef(ins, o->batch_offset());
    pushRef(outs, o->q_out());
    pushRef(outs, o->k_out());
    pushRef(outs, o->v_out());
    break;
  }
  case OpType::NLPConcatHeadsDecodeOp: {
    const auto *o = op->type_as_NLPConcatHeadsDecodeOp();
    pushRef(ins, o->in());
    pushRef(outs, o->out());
    break;
  }
  case OpType::RotaryEmbeddingLlamaOp: {
    const auto *o = op->type_as_RotaryEmbeddingLlamaOp();
    pushRef(ins, o->input());
    pushRef(ins, o->cos_cache());
    pushRef(ins, o->sin_cache());
    pushRef(ins, o->trans_mat());
    pushRef(outs, o->out());
    break;
  }
  case OpType::MaxPool2dWithIndicesOp: {
    const auto *o = op->type_as_MaxPool2dWithIndicesOp();
    pushRef(ins, o->in());
    pushRef(outs, o->result());
    pushRef(outs, o->result_indices());
    break;
  }
  case OpType::DropoutOp: {
    const auto *o = op->type_as_DropoutOp();
    pushRef(ins, o->in());
    pushRef(outs, o->out());
    break;
  }
  case OpType::RandOp: pushRef(outs, op->type_as_RandOp()->out()); break;
  case OpType::BatchNormTrainingOp: {
    const auto *o = op->type_as_BatchNormTrainingOp();
    pushRef(ins, o->input());
    pushRef(ins, o->running_mean());
    pushRef(ins, o->running_var());
    pushRef(ins, o->weight());
    pushRef(ins, o->bias());
    pushRef(outs, o->out());
    break;
  }
  case OpType::GroupNormOp: {
    const auto *o = op->type_as_GroupNormOp();
    pushRef(ins, o->input());
    pushRef(ins, o->input_mask());
    pushRef(ins, o->weight());
    pushRef(ins, o->bias());
    pushRef(outs, o->out());
    break;
  }
  case OpType::ConvTranspose2dOp: {
    const auto *o = op->type_as_ConvTranspose2dOp();
    pushRef(ins, o->input());
    pushRef(ins, o->weight());
    pushRef(ins, o->bias());
    pushRef(outs, o->out());
    break;
  }
  case OpType::Conv1dOp: {
    const auto *o = op->type_as_Conv1dOp();
    pushRef(ins, o->input());
    pushRef(ins, o->weight());
    pushRef(ins, o->bias());
    pushRef(outs, o->out());
    break;
  }
  case OpType::BatchNormInferenceOp: {
    const auto *o = op->type_as_BatchNormInferenceOp();
    pushRef(ins, o->input());
    pushRef(ins, o->running_mean());
    pushRef(ins, o->running_var());
    pushRef(ins, o->weight());
    pushRef(ins, o->bias());
    pushRef(outs, o->out());
    break;
  }
  case OpType::LayerNormOp: {
    const auto *o = op->type_as_LayerNormOp();
    pushRef(ins, o->input());
    pushRef(ins, o->weight());
    pushRef(ins, o->bias());
    pushRef(outs, o->out());
    break;
  }
  case OpType::FillCacheOp: {
    const auto *o = op->type_as_FillCacheOp();
    pushRef(ins, o->cache());
    pushRef(ins, o->input());
    break;
  }
  case OpType::UpdateCacheOp: {
    const auto *o = op->type_as_UpdateCacheOp();
    pushRef(ins, o->cache());
    pushRef(ins, o->input());
    pushRef(ins, o->update_index());
    break;
  }
  case OpType::ScaledDotProductAttentionDecodeOp: {
    const auto *o = op->type_as_ScaledDotProductAttentionDecodeOp();
    pushRef(ins, o->query());
    pushRef(ins, o->key());
    pushRef(ins, o->value());
    pushRef(ins, o->attention_mask());
    pushRef(ins, o->cur_pos_tensor());
    pushRef(ins, o->attention_sink());
    pushRef(outs, o->out());
    break;
  }
  case OpType::EmbeddingOp: {
    const auto *o = op->type_as_EmbeddingOp();
    pushRef(ins, o->input());
    pushRef(ins, o->weight());
    pushRef(outs, o->out());
    break;
  }
  case OpType::GatherOp: {
    const auto *o = op->type_as_GatherOp();
    pushRef(ins, o->input());
    pushRef(ins, o->index());
    pushRef(outs, o->out());
    break;
  }
  case OpType::ScatterOp: {
    const auto *o = op->type_as_ScatterOp();
    pushRef(ins, o->input());
    pushRef(ins, o->index());
    pushRef(ins, o->source());
    pushRef(outs, o->out());
    break;
  }
  case OpType::SortOp: {
    const auto *o = op->type_as_SortOp();
    pushRef(ins, o->in());
    if (o->outputs()) {
      for (const auto *r : *o->outputs()) pushRef(outs, r);
    }
    break;
  }
  case OpType::TopKOp: {
    const auto *o = op->type_as_TopKOp();
    pushRef(ins, o->input_tensor());
    if (o->outputs()) {
      for (const auto *r : *o->outputs()) pushRef(outs, r);
    }
    break;
  }
  case OpType::SamplingOp: {
    const auto *o = op->type_as_SamplingOp();
    pushRef(ins, o->input_values());
    pushRef(ins, o->input_indices());
    pushRef(ins, o->k());
    pushRef(ins, o->p());
    pushRef(ins, o->temp());
    pushRef(outs, o->out());
    break;
  }
  case OpType::PagedUpdateCacheOp: {
    const auto *o = op->type_as_PagedUpdateCacheOp();
    pushRef(ins, o->cache());
    pushRef(ins, o->input());
    pushRef(ins, o->update_index());
    pushRef(ins, o->page_table());
    break;
  }
  case OpType::PagedFillCacheOp: {
    const auto *o = op->type_as_PagedFillCacheOp();
    pushRef(ins, o->cache());
    pushRef(ins, o->input());
    pushRef(ins, o->page_table());
    pushRef(ins, o->batch_idx_tensor());
    break;
  }
  case OpType::PagedScaledDotProductAttentionDecodeOp: {
    const auto *o = op->type_as_PagedScaledDotProductAttentionDecodeOp();
    pushRef(ins, o->query());
    pushRef(ins, o->key());
    pushRef(ins, o->value());
    pushRef(ins, o->page_table());
    pushRef(ins, o->attention_mask());
    pushRef(ins, o->cur_pos_tensor());
    pushRef(ins, o->attention_sink());
    pushRef(outs, o->out());
    break;
  }
  case OpType::EltwiseBinaryOp: {
    const auto *o = op->type_as_EltwiseBinaryOp();
    pushRef(ins, o->lhs());
    pushRef(ins, o->rhs());
    pushRef(outs, o->out());
    break;
  }
  case OpType::EltwiseBinaryCompositeOp: {
    const auto *o = op->type_as_EltwiseBinaryCompositeOp();
    pushRef(ins, o->lhs());
    pushRef(ins, o->rhs());
    pushRef(outs, o->out());
    break;
  }
  case OpType::EltwiseTernaryWhereOp: {
    const auto *o = op->type_as_EltwiseTernaryWhereOp();
    pushRef(ins, o->first());
    pushRef(ins, o->second());
    pushRef(ins, o->third());
    pushRef(outs, o->out());
    break;
  }
  case OpType::EltwiseQuantizationOp: {
    const auto *o = op->type_as_EltwiseQuantizationOp();
    pushRef(ins, o->in());
    quantParamRefs(o, ins);
    pushRef(outs, o->out());
    break;
  }
  case OpType::MatmulOp: {
    const auto *o = op->type_as_MatmulOp();
    pushRef(ins, o->a());
    pushRef(ins, o->b());
    pushRef(outs, o->out());
    break;
  }
  case OpType::LinearOp: {
    const auto *o = op->type_as_LinearOp();
    pushRef(ins, o->a());
    pushRef(ins, o->b());
    pushRef(ins, o->bias());
    pushRef(outs, o->out());
    break;
  }
  case OpType::Conv2dOp: {
    const auto *o = op->type_as_Conv2dOp();
    pushRef(ins, o->input());
    pushRef(ins, o->weight());
    pushRef(ins, o->bias());
    pushRef(outs, o->out());
    break;
  }
  case OpType::RMSNormOp: {
    const auto *o = op->type_as_RMSNormOp();
    pushRef(ins, o->input());
    pushRef(ins, o->weight());
    pushRef(ins, o->bias());
    pushRef(outs, o->out());
    break;
  }
  case OpType::ConcatOp: {
    const auto *o = op->type_as_ConcatOp();
    if (o->inputs()) {
      for (const auto *r : *o->inputs()) pushRef(ins, r);
    }
    pushRef(outs, o->out());
    break;
  }
  case OpType::RotaryEmbeddingOp: {
    const auto *o = op->type_as_RotaryEmbeddingOp();
    pushRef(ins, o->input());
    pushRef(ins, o->cos_cache());
    pushRef(ins, o->sin_cache());
    pushRef(outs, o->out());
    break;
  }
  case OpType::ScaledDotProductAttentionOp: {
    const auto *o = op->type_as_ScaledDotProductAttentionOp();
    pushRef(ins, o->query());
    pushRef(ins, o->key());
    pushRef(ins, o->value());
    pushRef(ins, o->attention_mask());
    pushRef(ins, o->attention_sink());
    pushRef(outs, o->out());
    break;
  }
  case OpType::SplitQueryKeyValueAndSplitHeadsOp: {
    const auto *o = op->type_as_SplitQueryKeyValueAndSplitHeadsOp();
    pushRef(ins, o->in());
    pushRef(ins, o->kv_input());
    pushRef(outs, o->q_out());
    pushRef(outs, o->k_out());
    pushRef(outs, o->v_out());
    break;
  }
  case OpType::DeallocateOp:
    pushRef(ins, op->type_as_DeallocateOp()->in());
    break;
  case OpType::CpuOp: {
    const auto *o = op->type_as_CpuOp();
    if (o->ins()) for (const auto *r : *o->ins()) pushRef(ins, r);
    if (o->outs()) for (const auto *r : *o->outs()) pushRef(outs, r);
    break;
  }
  case OpType::LoadCachedOp: {
    const auto *o = op->type_as_LoadCachedOp();
    if (o->inputs()) for (const auto *r : *o->inputs()) pushRef(ins, r);
    if (o->outputs()) for (const auto *r : *o->outputs()) pushRef(outs, r);
    break;
  }
  case OpType::FuncCallOp: {
    const auto *o = op->type_as_FuncCallOp();
    if (o->inputs()) for (const auto *r : *o->inputs()) pushRef(ins, r);
    if (o->outputs()) for (const auto *r : *o->outputs()) pushRef(outs, r);
    break;
  }
  case OpType::CaptureOrExecuteTraceOp: {
    const auto *o = op->type_as_CaptureOrExecuteTraceOp();
    if (o->inputs()) for (const auto *r : *o->inputs()) pushRef(ins, r);
    if (o->outputs()) for (const auto *r : *o->outputs()) pushRef(outs, r);
    break;
  }
  case OpType::BeginTraceCaptureOp: pushRef(outs, op->type_as_BeginTraceCaptureOp()->trace_id()); break;
  case OpType::EndTraceCaptureOp: pushRef(ins, op->type_as_EndTraceCaptureOp()->trace_id()); break;
  case OpType::ExecuteTraceOp: pushRef(ins, op->type_as_ExecuteTraceOp()->trace_id()); break;
  case OpType::WriteTensorOp: {
    const auto *o = op->type_as_WriteTensorOp();
    pushRef(ins, o->host_tensor());
    pushRef(ins, o->device_tensor());
    break;
  }
  case OpType::CopyOp: {
    const auto *o = op->type_as_CopyOp();
    pushRef(ins, o->src());
    pushRef(ins, o->dst());
    break;
  }
  case OpType::ArangeOp: pushRef(outs, op->type_as_ArangeOp()->out()); break;
  case OpType::ConstantOp: pushRef(outs, op->type_as_ConstantOp()->out()); break;
  case OpType::EmptyOp: pushRef(outs, op->type_as_EmptyOp()->out()); break;
  case OpType::FullOp: pushRef(outs, op->type_as_FullOp()->out()); break;
  case OpType::NamedFullOp: pushRef(outs, op->type_as_NamedFullOp()->out()); break;
  default:
    break;
  }
}

// Computed per submit: one pass over the op list (microseconds), so nothing keyed by a binary's
// address can go stale when a buffer is freed and its address reused by another binary.
static ProgramInfo programInfo(const fbt::Program *prog) {
  ProgramInfo info;
  if (prog->outputs()) {
    for (const auto *r : *prog->outputs()) info.outputs.insert(r->global_id());
  }
  if (prog->operations()) {
    std::vector<const fbt::TensorRef *> ins, outs;
    uint32_t index = 0;
    for (const auto *op : *prog->operations()) {
      uint32_t at = index++;
      if (op->type_type() == OpType::DeallocateOp) continue;
      ins.clear();
      outs.clear();
      collectOpRefs(op, ins, outs);
      for (const auto *r : ins) {
        info.useCount[r->global_id()]++;
        info.firstUse.emplace(r->global_id(), at);
      }
      if (const auto *cp = op->type_as_CopyOp()) {
        if (cp->src() && cp->dst()) info.copyTarget.emplace(cp->src()->global_id(), cp->dst());
      }
    }
  }
  return info;
}

// ---- helpers over TensorRef -----------------------------------------------------------------
static std::vector<uint32_t> refShape(const fbt::TensorRef *ref) {
  std::vector<uint32_t> s;
  TTRT_ASSERT(ref && ref->desc(), "tensor ref has no descriptor");
  if (ref->desc()->shape()) {
    for (int32_t d : *ref->desc()->shape()) {
      TTRT_ASSERT(d >= 0, "negative dimension in tensor ", ref->global_id());
      s.push_back(static_cast<uint32_t>(d));
    }
  }
  return s;
}

static DataType refDtype(const fbt::TensorRef *ref) {
  TTRT_ASSERT(ref && ref->desc() && ref->desc()->layout() && ref->desc()->layout()->memory_desc(),
              "tensor ref has no memory descriptor");
  return ref->desc()->layout()->memory_desc()->data_type();
}

static bool refOnDevice(const fbt::TensorRef *ref) {
  return ref->desc()->layout()->memory_desc()->storage_type() == fbt::StorageType::Device;
}

static TensorLayout refLayout(const fbt::TensorRef *ref) {
  const auto *ts = ref->desc()->layout()->memory_desc()->tile_shape();
  return (ts && ts->y() == 32 && ts->x() == 32) ? TensorLayout::Tile : TensorLayout::RowMajor;
}

static int normDim(int64_t d, size_t rank) {
  int64_t r = static_cast<int64_t>(rank);
  if (d < 0) d += r;
  TTRT_ASSERT(d >= 0 && d < std::max<int64_t>(r, 1), "dimension ", d, " out of range for rank ", rank);
  return static_cast<int>(d);
}

static size_t prod(const std::vector<uint32_t> &s, size_t from, size_t to) {
  size_t v = 1;
  for (size_t i = from; i < to && i < s.size(); ++i) v *= s[i];
  return v;
}

static float numberValue(fbt::NumberType ty, const void *p) {
  if (ty == fbt::NumberType::FP) return static_cast<const fbt::FloatingPointType *>(p)->value();
  if (ty == fbt::NumberType::I32) return static_cast<float>(static_cast<const fbt::IntegralType *>(p)->value());
  return 0.0f;
}

static int activationCode(const fb::String *s) {
  if (!s || s->size() == 0) return TTB_ACT_NONE;
  std::string_view v = s->view();
  if (v == "relu") return TTB_ACT_RELU;
  if (v == "silu") return TTB_ACT_SILU;
  if (v == "gelu") return TTB_ACT_GELU;
  if (v == "sigmoid") return TTB_ACT_SIGMOID;
  TTRT_FATAL("unsupported fused activation '", std::string(v), "'");
}

// ---- the executor -----------------------------------------------------------------------------
struct ProgramContextImpl;

class Executor {
public:
  Executor(std::shared_ptr<DeviceImpl> dev, Binary &bin, uint32_t programIndex, std::vector<Tensor> &inputs);
  std::vector<Tensor> run();

  // used by the hook API
  std::unordered_map<uint32_t, TensorPtr> pool;
  uint32_t programIndex;
  std::shared_ptr<DeviceImpl> dev;

private:
  Binary &bin;
  const fbt::Program *prog = nullptr;
  ProgramInfo info;
  bool fuse = true;
  // A head split ([B,S,H,D] -> [B,H,S,D] permute) whose only consumer reads through strides
  // (rotary embedding, attention) is not materialised: the consumer gets the source tensor and
  // the permuted strides.  Any other access (get) performs the copy after all.
  struct LazyView {
    TensorPtr base;
    std::vector<uint32_t> shape;
    std::vector<int64_t> strides; // in elements, over `shape`
  };
  std::unordered_map<uint32_t, LazyView> lazy;
  // Inputs of rotary_embedding ops whose rotation the producing projection has already applied.
  std::unordered_set<uint32_t> ropeApplied;
  // Dense strides of a live tensor, or the pending view of `ref`, as {tensor, strides}.
  std::pair<TensorPtr, std::vector<int64_t>> viewOf(const fbt::TensorRef *ref);

  TensorPtr get(const fbt::TensorRef *ref);
  TensorPtr getDevice(const fbt::TensorRef *ref); // uploads a host tensor if an op needs it on device
  void put(const fbt::TensorRef *ref, TensorPtr t);
  TensorPtr allocOut(const fbt::TensorRef *ref);
  bool singleUse(const fbt::TensorRef *ref) const;
  template <typename F> void eachRank(F &&f);

  size_t runOp(size_t i); // returns the number of ops consumed
  // Next op at or after `from` that is not a DeallocateOp; records the skipped deallocations.
  const fbt::Operation *peek(size_t &idx, std::vector<const fbt::Operation *> &skipped) const;
  void runDeallocs(const std::vector<const fbt::Operation *> &ops);

  // fused forms; return ops consumed or 0 when the pattern does not apply
  size_t tryQuantChain(size_t i);
  size_t tryGemmEpilogue(size_t i);
  size_t tryQuantizedGemm(size_t i);
  size_t tryQuantizedConv(size_t i);
  TensorPtr convDeqScale;     // set around runConv2d by tryQuantizedConv: the fused dequantize's per-channel scale
  float convDeqScalar = 0.0f; // ... or its per-tensor scale
  // matmul on quantized (8-bit integer) operands; deqScale / deqScalar describe a fused dequantize
  void runIntGemm(const fbt::TensorRef *aRef, const fbt::TensorRef *bRef, const fbt::TensorRef *outRef, bool ta, bool tb,
                  const TensorPtr &deqScale, float deqScalar, const fbt::TensorRef *biasRef = nullptr);
  size_t tryGroupedGemm(size_t i);
  const fbt::RotaryEmbeddingOp *ropeAfter(const fbt::TensorRef *out) const;
  size_t trySwiglu(size_t i);
  size_t trySiluMul(size_t i);
  size_t trySdpa(size_t i);
  size_t tryAllReduceAdd(size_t i);
  bool symmReady(size_t bytes);
  TensorPtr allocForAllReduce(const fbt::TensorRef *ref); // null unless `ref` feeds the next all-reduce
  bool feedsSymmAllReduce(const fbt::TensorRef *ref);      // `ref`'s only consumer is an all-reduce the peer-memory kernel takes
  // GEMM whose result only feeds an all-reduce: scattered into the peers' workspaces.  Null = not applicable.
  TensorPtr tryGemmPush(const TensorPtr &a, const TensorPtr &b, const fbt::TensorRef *outRef, int64_t M, int64_t N, int64_t K);
  size_t curOp = 0;
  void allReduce(const TensorPtr &in, const TensorPtr &residual, const TensorPtr &out, int reduceType);
  size_t tryAddRmsNorm(size_t i);

  void runGetDevice(const fbt::GetDeviceOp *op);
  void runToDevice(const fbt::ToDeviceOp *op);
  void runFromDevice(const fbt::FromDeviceOp *op);
  void runToLayout(const fbt::ToLayoutOp *op);
  void runToMemoryConfig(const fbt::ToMemoryConfigOp *op);
  void runTypecast(const fbt::TypecastOp *op);
  void runDeallocate(const fbt::DeallocateOp *op);
  void runFull(const fbt::FullOp *op);
  void runNamedFull(const fbt::NamedFullOp *op);
  void runConstant(const fbt::ConstantOp *op);
  void runEmpty(const fbt::EmptyOp *op);
  void runArange(const fbt::ArangeOp *op);
  void runUnary(const fbt::EltwiseUnaryOp *op);
  void runUnaryComposite(const fbt::EltwiseUnaryCompositeOp *op);
  void runBinary(int opCode, const fbt::TensorRef *lhs, const fbt::TensorRef *rhs, const fbt::TensorRef *out);
  void runWhere(const fbt::EltwiseTernaryWhereOp *op);
  void runQuantization(const fbt::EltwiseQuantizationOp *op);
  void runGemm(const fbt::TensorRef *a, const fbt::TensorRef *b, const fbt::TensorRef *bias, const fbt::TensorRef *out,
               bool ta, bool tb, int act, int roundSteps, const fbt::TensorRef *extra = nullptr, int extraOp = 0);
  void runConv2d(const fbt::Conv2dOp *op, int act = 0, const fbt::TensorRef *extra = nullptr, int extraOp = 0,
                 const fbt::TensorRef *outRef = nullptr);
  size_t tryConvEpilogue(size_t i);
  size_t tryPointwisePair(size_t i);
  void runSoftmax(const fbt::SoftmaxOp *op);
  void runRmsNorm(const fbt::RMSNormOp *op);
  void runReduction(const fbt::ReductionOp *op);
  void runReshape(const fbt::ReshapeOp *op);
  void runPermute(const fbt::TensorRef *in, const std::vector<int> &perm, const fbt::TensorRef *out);
  void runConcat(const fbt::ConcatOp *op);
  void runSlice(const fbt::SliceOp *op);
  void runRepeat(const fbt::RepeatOp *op);
  void runRepeatInterleave(const fbt::RepeatInterleaveOp *op);
  void runConcatenateHeads(const fbt::ConcatenateHeadsOp *op);
  void runSplitQkv(const fbt::SplitQueryKeyValueAndSplitHeadsOp *op);
  void runRotaryEmbedding(const fbt::RotaryEmbeddingOp *op);
  void runSdpa(const fbt::ScaledDotProductAttentionOp *op);
  void runAllReduce(const fbt::AllReduceOp *op);
  void runAllGather(const fbt::AllGatherOp *op);
  void runReduceScatter(const fbt::ReduceScatterOp *op);
  void runMeshPartition(const fbt::MeshPartitionOp *op);
  void runDistribute(const fbt::DistributeTensorOp *op);
  void runAggregate(const fbt::AggregateTensorOp *op);
  void runLayerNorm(const fbt::LayerNormOp *op);
  void runArgMax(const fbt::ReductionArgMaxOp *op);
  void runCumSum(const fbt::CumSumOp *op);
  void runCumProd(const fbt::CumProdOp *op);
  // expert ownership of this process's mesh coordinates: localIdx tensors (Int32 [experts]) from a [1, 1, E, D] mapping
  TensorPtr moeLocalIndex(const TensorPtr &mapping, uint32_t &experts, uint32_t &devices);
  void runAllToAllDispatch(const fbt::AllToAllDispatchOp *op);
  void runPagedMlaDecode(const fbt::PagedFlashMultiLatentAttentionDecodeOp *op);
  void runFlashMlaPrefill(const fbt::FlashMlaPrefillOp *op);
  void runIndexerScoreDsa(const fbt::IndexerScoreDsaOp *op);
  void runChunkedSdpa(const fbt::ChunkedScaledDotProductAttentionOp *op);
  void runConv3d(const fbt::Conv3dOp *op);
  void runGeluBackward(const fbt::ExperimentalEltwiseBinaryBackwardOp *op);
  void runEmbeddingBackward(const fbt::EmbeddingBackwardOp *op);
  void runAdamW(const fbt::AdamWOp *op);
  void runAllToAllDispatchMetadata(const fbt::AllToAllDispatchMetadataOp *op);
  void runTopKRouterGpt(const fbt::TopKRouterGptOp *op);
  void runAllToAllCombine(const fbt::AllToAllCombineOp *op);
  void runMoeExpertTokenRemap(const fbt::MoeExpertTokenRemapOp *op);
  void runSparseMatmul(const fbt::SparseMatmulOp *op);
  void runDitRmsNorm(const fbt::DitRMSNormUnaryFusedOp *op);
  void runDistributedRmsNorm(const fbt::DistributedRMSNormOp *op);
  void runNormPreAllGather(const fbt::TensorRef *in, const fbt::TensorRef *residual, const fbt::TensorRef *out, int mode);
  void runLayerNormPostAllGather(const fbt::LayerNormPostAllGatherOp *op);
  void runAssign(const fbt::AssignOp *op);
  void runPowScalar(const fbt::EltwiseBinaryCompositeScalarOp *op);
  void runDumpTensor(const fbt::DumpTensorOp *op);
  void runLoadTensor(const fbt::LoadTensorOp *op);
  void runAlias(const fbt::TensorRef *operand, const fbt::TensorRef *result);
  void runMemorySnapshot(const fbt::MemorySnapshotOp *op);
  void runAllReduceAsync(const fbt::AllReduceAsyncOp *op);
  void runPointToPoint(const fbt::PointToPointOp *op);
  void runNlpCreateQkvHeadsDecode(const fbt::NLPCreateQKVHeadsDecodeOp *op);
  void runNlpConcatHeadsDecode(const fbt::NLPConcatHeadsDecodeOp *op);
  void runRotaryEmbeddingLlama(const fbt::RotaryEmbeddingLlamaOp *op);
  void runMaxPool2dWithIndices(const fbt::MaxPool2dWithIndicesOp *op);
  void runDropout(const fbt::DropoutOp *op);
  void runRand(const fbt::RandOp *op);
  void runBatchNormTraining(const fbt::BatchNormTrainingOp *op);
  void runGroupNorm(const fbt::GroupNormOp *op);
  void runConvTranspose2d(const fbt::ConvTranspose2dOp *op);
  void runConv1d(const fbt::Conv1dOp *op);
  void runBitcastConvert(const fbt::BitcastConvertOp *op);
  void runNlpConcatHeads(const fbt::NLPConcatHeadsOp *op);
  void runReductionProd(const fbt::ReductionProdOp *op);
  void runBatchNormInference(const fbt::BatchNormInferenceOp *op);
  void runUpsample(const fbt::UpsampleOp *op);
  void runPrepareConv2d(const fbt::TensorRef *in, const fbt::TensorRef *out);
  void runEmbedding(const fbt::EmbeddingOp *op);
  void runGather(const fbt::GatherOp *op);
  void runScatter(const fbt::ScatterOp *op);
  void runSort(const fbt::SortOp *op);
  void runTopK(const fbt::TopKOp *op);
  // values / indices of the first `take` entries of x sorted along `dim` (shared by sort and top-k)
  void sortAlong(const TensorPtr &x, int dim, bool descending, size_t take, const fbt::TensorRef *valuesRef,
                 const fbt::TensorRef *indicesRef);
  void runSampling(const fbt::SamplingOp *op);
  void runPagedUpdateCache(const fbt::PagedUpdateCacheOp *op);
  void runPagedFillCache(const fbt::PagedFillCacheOp *op);
  void runPagedSdpaDecode(const fbt::PagedScaledDotProductAttentionDecodeOp *op);
  void runPool2d(const fbt::Pool2dOp *op);
  void runGlobalAvgPool2d(const fbt::GlobalAvgPool2dOp *op);
  void runPad(const fbt::PadOp *op);
  void runFillCache(const fbt::FillCacheOp *op);
  void runUpdateCache(const fbt::UpdateCacheOp *op);
  void runSdpaDecode(const fbt::ScaledDotProductAttentionDecodeOp *op);
  // sub-programs: const-eval cache, calls, traces
  std::vector<TensorPtr> runSubProgram(uint32_t index, const std::vector<TensorPtr> &inputs);
  void runLoadCached(const fbt::LoadCachedOp *op);
  void runFuncCall(const fbt::FuncCallOp *op);
  void runBeginTraceCapture(const fbt::BeginTraceCaptureOp *op);
  void runEndTraceCapture(const fbt::EndTraceCaptureOp *op);
  void runExecuteTrace(const fbt::ExecuteTraceOp *op);
  void runCaptureOrExecuteTrace(const fbt::CaptureOrExecuteTraceOp *op);
  void updateTraceInputSlots(const fbt::CaptureOrExecuteTraceOp *op, std::vector<TensorPtr> &slots, bool residentOnly);
  void runWriteTensor(const fbt::WriteTensorOp *op);
  void runCopy(const fbt::CopyOp *op);
  void refuseWhileRecording(const char *what) const;

  // gather-copy of a strided view of `in` into a new dense tensor shaped like `outShape`
  TensorPtr stridedView(const TensorPtr &in, const std::vector<uint32_t> &outShape, const std::vector<int64_t> &inStrides,
                        int64_t offset, DataType dt);
  uint32_t meshAxisSize(uint32_t clusterAxis) const;
};

struct ProgramContextImpl {
  Executor *executor;
};

Executor::Executor(std::shared_ptr<DeviceImpl> d, Binary &b, uint32_t pi, std::vector<Tensor> &inputs)
    : programIndex(pi), dev(std::move(d)), bin(b) {
  const auto *programs = bin.get()->programs();
  TTRT_ASSERT(programs && programIndex < programs->size(), "program index ", programIndex, " out of range");
  prog = programs->Get(programIndex);
  info = programInfo(prog);
  const auto &hooks = debug::Hooks::get();
  fuse = !debug::Env::get().disableFusion && !hooks.getPreOperatorCallback() && !hooks.getPostOperatorCallback();

  auto mesh = bin.getProgramMeshShape(programIndex);
  TTRT_ASSERT(mesh.first * mesh.second == dev->worldSize, "program was compiled for a ", mesh.first, "x", mesh.second,
              " mesh but the device has ", dev->worldSize, " chips");
  if (prog->dylibs() && prog->dylibs()->size() > 0) {
    logDebug("program embeds CPU dylibs; CpuOp is rejected by this target");
  }
  uint32_t nIn = prog->inputs() ? prog->inputs()->size() : 0;
  TTRT_ASSERT(inputs.size() == nIn, "program expects ", nIn, " inputs, got ", inputs.size());
  for (uint32_t i = 0; i < nIn; ++i) {
    const auto *ref = prog->inputs()->Get(i);
    TensorPtr t = unwrapTensor(inputs[i]);
    TTRT_ASSERT(t->allocated(), "input ", i, " has been deallocated");
    std::vector<uint32_t> want = refShape(ref);
    TTRT_ASSERT(t->volume() == prod(want, 0, want.size()), "input ", i, " has ", t->volume(), " elements, program expects ",
                prod(want, 0, want.size()));
    if (refOnDevice(ref) && t->storage == Storage::Host) {
      // The reference requires callers to run toLayout first; accepting a host tensor here
      // and uploading it is a convenience and costs one copy per submit.
      t = toDevice(t, dev, refDtype(ref));
    }
    TTRT_ASSERT(t->dtype == refDtype(ref), "input ", i, " has data type ", dataTypeName(t->dtype), ", program expects ",
                dataTypeName(refDtype(ref)));
    orderAfterUploads(t); // an upload still in flight on the copy stream: the compute stream waits for it
    if (t->shape != want) {
      // same volume, different view (for example a flattened activation)
      auto view = std::make_shared<TensorImpl>();
      view->shape = want;
      view->stride = denseStrides(want);
      view->dtype = t->dtype;
      view->storage = t->storage;
      view->layout = t->layout;
      view->shards = t->shards;
      view->device = t->device;
      view->retain = true;
      view->base = t->base ? t->base : t;
      view->version.store(view->base->version.load());
      t = view;
    }
    pool[ref->global_id()] = t;
  }
}

template <typename F> void Executor::eachRank(F &&f) {
  for (size_t i = 0; i < dev->locals.size(); ++i) {
    const RankCtx &r = dev->locals[i];
    if (dev->locals.size() > 1 || i == 0) {
      TTB_CALL(ttb_set_device(r.cudaDevice));
    }
    f(i, r);
  }
}

TensorPtr Executor::get(const fbt::TensorRef *ref) {
  TTRT_ASSERT(ref != nullptr, "missing tensor operand");
  auto lz = lazy.find(ref->global_id());
  if (lz != lazy.end()) {
    LazyView v = std::move(lz->second);
    lazy.erase(lz);
    pool[ref->global_id()] = stridedView(v.base, v.shape, v.strides, 0, v.base->dtype);
  }
  auto it = pool.find(ref->global_id());
  TTRT_ASSERT(it != pool.end(), "tensor ", ref->global_id(), " is not live (used before definition or after deallocation)");
  TTRT_ASSERT(it->second->allocated(), "tensor ", ref->global_id(), " has been deallocated");
  return it->second;
}

std::pair<TensorPtr, std::vector<int64_t>> Executor::viewOf(const fbt::TensorRef *ref) {
  TTRT_ASSERT(ref != nullptr, "missing tensor operand");
  auto lz = lazy.find(ref->global_id());
  if (lz != lazy.end()) return {lz->second.base, lz->second.strides};
  TensorPtr t = getDevice(ref);
  return {t, denseStrides(t->shape)};
}

TensorPtr Executor::getDevice(const fbt::TensorRef *ref) {
  TensorPtr t = get(ref);
  if (t->storage == Storage::Host) {
    refuseWhileRecording("a host-to-device copy");
    t = toDevice(t, dev, t->dtype);
    pool[ref->global_id()] = t;
  }
  return t;
}

void Executor::put(const fbt::TensorRef *ref, TensorPtr t) {
  TTRT_ASSERT(ref != nullptr, "op has no output ref");
  pool[ref->global_id()] = std::move(t);
}

TensorPtr Executor::allocOut(const fbt::TensorRef *ref) {
  auto ct = info.copyTarget.find(ref->global_id());
  if (ct != info.copyTarget.end() && singleUse(ref) && singleUse(ct->second)) {
    auto dst = pool.find(ct->second->global_id());
    // (retained: the DeallocateOp that follows the copy must not take the destination with it)
    if (dst != pool.end() && dst->second->storage == Storage::Device && dst->second->allocated() && dst->second->retain &&
        dst->second->dtype == refDtype(ref) && dst->second->shape == refShape(ref)) {
      return dst->second; // the CopyOp that follows finds source and destination identical
    }
  }
  auto t = makeDeviceTensor(dev, refShape(ref), refDtype(ref));
  t->layout = refLayout(ref);
  return t;
}

bool Executor::singleUse(const fbt::TensorRef *ref) const {
  uint32_t id = ref->global_id();
  auto it = info.useCount.find(id);
  return (it != info.useCount.end() && it->second == 1) && !info.outputs.count(id);
}

const fbt::Operation *Executor::peek(size_t &idx, std::vector<const fbt::Operation *> &skipped) const {
  const auto *ops = prog->operations();
  while (idx < ops->size() && ops->Get(idx)->type_type() == OpType::DeallocateOp) {
    skipped.push_back(ops->Get(idx));
    ++idx;
  }
  return idx < ops->size() ? ops->Get(idx) : nullptr;
}

void Executor::runDeallocs(const std::vector<const fbt::Operation *> &ops) {
  for (const auto *op : ops) {
    const auto *d = op->type_as_DeallocateOp();
    // Inside a fused chain an intermediate may never have been materialised.
    if (d->in() && (pool.count(d->in()->global_id()) || lazy.count(d->in()->global_id()))) runDeallocate(d);
  }
}

std::vector<Tensor> Executor::run() {
  const auto &hooks = debug::Hooks::get();
  auto ctxImpl = std::make_shared<ProgramContextImpl>();
  ctxImpl->executor = this;
  CallbackContext cbCtx(std::static_pointer_cast<void>(ctxImpl), DeviceRuntime::CUDA);
  if (hooks.getpreProgramCallback()) (*hooks.getpreProgramCallback())(bin, cbCtx);

  const auto *ops = prog->operations();
  size_t n = ops ? ops->size() : 0;
  bool syncAfterOp = debug::Env::get().syncAfterOp;
  perf::Env &perfEnv = perf::Env::get();
  const bool perfTrace = perfEnv.enablePerfTrace;
  // const-eval functions are the private programs the compiler names "<function>_const_eval_<n>"
  const bool constEvalProgram = prog->name() && prog->name()->str().find("const_eval") != std::string::npos;
  for (size_t i = 0; i < n;) {
    const auto *op = ops->Get(static_cast<uint32_t>(i));
    std::shared_ptr<OpContextImpl> opCtxImpl;
    if (hooks.getPreOperatorCallback() || hooks.getPostOperatorCallback()) {
      opCtxImpl = std::make_shared<OpContextImpl>();
      opCtxImpl->op = op;
    }
    if (hooks.getPreOperatorCallback()) {
      (*hooks.getPreOperatorCallback())(bin, cbCtx, OpContext(std::static_pointer_cast<void>(opCtxImpl), DeviceRuntime::CUDA));
    }
    size_t used;
    if (perfTrace) {
      // What the reference logs per op (runtime/lib/ttnn/program_executor.cpp:234-237), plus a range
      // named after the op that spans its launches (a fused chain is one range named after its first op).
      const std::string loc = op->loc_info() ? op->loc_info()->str() : "";
      perfEnv.tracyLogOpLocation(loc);
      perfEnv.tracyLogConstEvalProgram(constEvalProgram);
      perfEnv.tracyLogProgramMetadata(perfEnv.tracyProgramMetadata);
      perfEnv.rangePush(std::string(fbt::EnumNameOpType(op->type_type())) + " " + loc);
    }
    try {
      used = runOp(i);
    } catch (const std::runtime_error &e) {
      if (perfTrace) perfEnv.rangePop();
      std::string loc = op->loc_info() ? op->loc_info()->str() : "";
      throw std::runtime_error(std::string(e.what()) + " [while executing op #" + std::to_string(i) + " " +
                               fbt::EnumNameOpType(op->type_type()) + (loc.empty() ? "" : " at " + loc) + "]");
    }
    if (perfTrace) perfEnv.rangePop();
    if (syncAfterOp) {
      eachRank([&](size_t, const RankCtx &r) { TTB_CALL(ttb_stream_sync(r.stream)); });
    }
    if (hooks.getPostOperatorCallback()) {
      (*hooks.getPostOperatorCallback())(bin, cbCtx, OpContext(std::static_pointer_cast<void>(opCtxImpl), DeviceRuntime::CUDA));
    }
    i += used;
  }

  std::vector<Tensor> outs;
  if (prog->outputs()) {
    for (const auto *ref : *prog->outputs()) {
      TensorPtr t = get(ref);
      outs.push_back(wrapTensor(t));
    }
  }
  if (hooks.getpostProgramCallback()) (*hooks.getpostProgramCallback())(bin, cbCtx);
  return outs;
}

size_t Executor::runOp(size_t i) {
  const auto *op = prog->operations()->Get(static_cast<uint32_t>(i));
  curOp = i;
  if (fuse) {
    size_t used = 0;
    switch (op->type_type()) {
    case OpType::EltwiseQuantizationOp: used = tryQuantChain(i); break;
    case OpType::MatmulOp:
    case OpType::LinearOp:
      used = tryQuantizedGemm(i);
      if (!used) used = trySwiglu(i);
      if (!used) used = tryGemmEpilogue(i);
      if (!used) used = tryGroupedGemm(i);
      break;
    case OpType::EltwiseUnaryOp: used = trySiluMul(i); break;
    case OpType::EltwiseBinaryOp: used = tryAddRmsNorm(i); break;
    case OpType::ScaledDotProductAttentionOp: used = trySdpa(i); break;
    case OpType::AllReduceOp: used = tryAllReduceAdd(i); break;
    case OpType::Conv2dOp:
      used = tryQuantizedConv(i);
      if (!used) used = tryConvEpilogue(i);
      break;
    default: break;
    }
    if (used) return used;
  }
  switch (op->type_type()) {
  case OpType::GetDeviceOp: runGetDevice(op->type_as_GetDeviceOp()); break;
  case OpType::ToDeviceOp: runToDevice(op->type_as_ToDeviceOp()); break;
  case OpType::FromDeviceOp: runFromDevice(op->type_as_FromDeviceOp()); break;
  case OpType::ToLayoutOp: runToLayout(op->type_as_ToLayoutOp()); break;
  case OpType::ToMemoryConfigOp: runToMemoryConfig(op->type_as_ToMemoryConfigOp()); break;
  case OpType::TypecastOp: runTypecast(op->type_as_TypecastOp()); break;
  case OpType::DeallocateOp: runDeallocate(op->type_as_DeallocateOp()); break;
  case OpType::FullOp: runFull(op->type_as_FullOp()); break;
  case OpType::NamedFullOp: runNamedFull(op->type_as_NamedFullOp()); break;
  case OpType::ConstantOp: runConstant(op->type_as_ConstantOp()); break;
  case OpType::EmptyOp: runEmpty(op->type_as_EmptyOp()); break;
  case OpType::ArangeOp: runArange(op->type_as_ArangeOp()); break;
  case OpType::EltwiseUnaryOp: runUnary(op->type_as_EltwiseUnaryOp()); break;
  case OpType::EltwiseUnaryCompositeOp: runUnaryComposite(op->type_as_EltwiseUnaryCompositeOp()); break;
  case OpType::EltwiseBinaryOp: {
    const auto *o = op->type_as_EltwiseBinaryOp();
    runBinary(static_cast<int>(o->type()), o->lhs(), o->rhs(), o->out());
    break;
  }
  case OpType::EltwiseBinaryCompositeOp: {
    const auto *o = op->type_as_EltwiseBinaryCompositeOp();
    runBinary(TTB_BINARY_COMPOSITE_BASE + static_cast<int>(o->type()), o->lhs(), o->rhs(), o->out());
    break;
  }
  case OpType::EltwiseTernaryWhereOp: runWhere(op->type_as_EltwiseTernaryWhereOp()); break;
  case OpType::EltwiseQuantizationOp: runQuantization(op->type_as_EltwiseQuantizationOp()); break;
  case OpType::MatmulOp: {
    const auto *o = op->type_as_MatmulOp();
    runGemm(o->a(), o->b(), nullptr, o->out(), o->transpose_a(), o->transpose_b(), activationCode(o->activation()), 0);
    break;
  }
  case OpType::LinearOp: {
    const auto *o = op->type_as_LinearOp();
    runGemm(o->a(), o->b(), o->bias(), o->out(), o->transpose_a(), o->transpose_b(), activationCode(o->activation()), 0);
    break;
  }
  case OpType::Conv2dOp: runConv2d(op->type_as_Conv2dOp()); break;
  case OpType::SoftmaxOp: runSoftmax(op->type_as_SoftmaxOp()); break;
  case OpType::RMSNormOp: runRmsNorm(op->type_as_RMSNormOp()); break;
  case OpType::ReductionOp: runReduction(op->type_as_ReductionOp()); break;
  case OpType::ReshapeOp: runReshape(op->type_as_ReshapeOp()); break;
  case OpType::PermuteOp: {
    const auto *o = op->type_as_PermuteOp();
    std::vector<int> perm;
    TTRT_ASSERT(o->permutation(), "permute without permutation");
    for (int64_t p : *o->permutation()) perm.push_back(static_cast<int>(p));
    runPermute(o->in(), perm, o->out());
    break;
  }
  case OpType::TransposeOp: {
    const auto *o = op->type_as_TransposeOp();
    size_t rank = refShape(o->in()).size();
    std::vector<int> perm(rank);
    for (size_t k = 0; k < rank; ++k) perm[k] = static_cast<int>(k);
    std::swap(perm[normDim(o->dim0(), rank)], perm[normDim(o->dim1(), rank)]);
    runPermute(o->in(), perm, o->out());
    break;
  }
  case OpType::ConcatOp: runConcat(op->type_as_ConcatOp()); break;
  case OpType::SliceOp: runSlice(op->type_as_SliceOp()); break;
  case OpType::RepeatOp: runRepeat(op->type_as_RepeatOp()); break;
  case OpType::RepeatInterleaveOp: runRepeatInterleave(op->type_as_RepeatInterleaveOp()); break;
  case OpType::ConcatenateHeadsOp: runConcatenateHeads(op->type_as_ConcatenateHeadsOp()); break;
  case OpType::SplitQueryKeyValueAndSplitHeadsOp: runSplitQkv(op->type_as_SplitQueryKeyValueAndSplitHeadsOp()); break;
  case OpType::RotaryEmbeddingOp: runRotaryEmbedding(op->type_as_RotaryEmbeddingOp()); break;
  case OpType::ScaledDotProductAttentionOp: runSdpa(op->type_as_ScaledDotProductAttentionOp()); break;
  case OpType::AllReduceOp: runAllReduce(op->type_as_AllReduceOp()); break;
  case OpType::AllGatherOp: runAllGather(op->type_as_AllGatherOp()); break;
  case OpType::ReduceScatterOp: runReduceScatter(op->type_as_ReduceScatterOp()); break;
  case OpType::MeshPartitionOp: runMeshPartition(op->type_as_MeshPartitionOp()); break;
  case OpType::DistributeTensorOp: runDistribute(op->type_as_DistributeTensorOp()); break;
  case OpType::AggregateTensorOp: runAggregate(op->type_as_AggregateTensorOp()); break;
  case OpType::LayerNormOp: runLayerNorm(op->type_as_LayerNormOp()); break;
  case OpType::ReductionArgMaxOp: runArgMax(op->type_as_ReductionArgMaxOp()); break;
  case OpType::CumSumOp: runCumSum(op->type_as_CumSumOp()); break;
  case OpType::CumProdOp: runCumProd(op->type_as_CumProdOp()); break;
  case OpType::AllToAllDispatchOp: runAllToAllDispatch(op->type_as_AllToAllDispatchOp()); break;
  case OpType::PagedFlashMultiLatentAttentionDecodeOp: runPagedMlaDecode(op->type_as_PagedFlashMultiLatentAttentionDecodeOp()); break;
  case OpType::FlashMlaPrefillOp: runFlashMlaPrefill(op->type_as_FlashMlaPrefillOp()); break;
  case OpType::IndexerScoreDsaOp: runIndexerScoreDsa(op->type_as_IndexerScoreDsaOp()); break;
  case OpType::ChunkedScaledDotProductAttentionOp: runChunkedSdpa(op->type_as_ChunkedScaledDotProductAttentionOp()); break;
  case OpType::Conv3dOp: runConv3d(op->type_as_Conv3dOp()); break;
  case OpType::PrepareConv3dWeightsOp: {
    const auto *o = op->type_as_PrepareConv3dWeightsOp();
    runPrepareConv2d(o->weight_tensor(), o->out());
    break;
  }
  case OpType::ExperimentalEltwiseBinaryBackwardOp: runGeluBackward(op->type_as_ExperimentalEltwiseBinaryBackwardOp()); break;
  case OpType::EmbeddingBackwardOp: runEmbeddingBackward(op->type_as_EmbeddingBackwardOp()); break;
  case OpType::AdamWOp: runAdamW(op->type_as_AdamWOp()); break;
  case OpType::AllToAllDispatchMetadataOp: runAllToAllDispatchMetadata(op->type_as_AllToAllDispatchMetadataOp()); break;
  case OpType::TopKRouterGptOp: runTopKRouterGpt(op->type_as_TopKRouterGptOp()); break;
  case OpType::AllToAllCombineOp: runAllToAllCombine(op->type_as_AllToAllCombineOp()); break;
  case OpType::MoeExpertTokenRemapOp: runMoeExpertTokenRemap(op->type_as_MoeExpertTokenRemapOp()); break;
  case OpType::SparseMatmulOp: runSparseMatmul(op->type_as_SparseMatmulOp()); break;
  case OpType::DitRMSNormUnaryFusedOp: runDitRmsNorm(op->type_as_DitRMSNormUnaryFusedOp()); break;
  case OpType::DistributedRMSNormOp: runDistributedRmsNorm(op->type_as_DistributedRMSNormOp()); break;
  case OpType::RMSNormPreAllGatherOp: {
    const auto *o = op->type_as_RMSNormPreAllGatherOp();
    runNormPreAllGather(o->input(), o->residual(), o->out(), 0);
    break;
  }
  case OpType::LayerNormPreAllGatherOp: {
    const auto *o = op->type_as_LayerNormPreAllGatherOp();
    runNormPreAllGather(o->input(), o->residual_input(), o->out(), 1); // `recip` is a lookup table of the Tensix kernel
    break;
  }
  case OpType::LayerNormPostAllGatherOp: runLayerNormPostAllGather(op->type_as_LayerNormPostAllGatherOp()); break;
  // Global semaphores synchronise Tensix cores of the reference's collectives (operations/global_semaphore/); the
  // collectives here order themselves on the stream, so the ops have nothing to create or reset.
  case OpType::CreateGlobalSemaphoreOp:
  case OpType::ResetGlobalSemaphoreOp:
  case OpType::AllocateMoeComputeSemaphoreOp: break;
  case OpType::AssignOp: runAssign(op->type_as_AssignOp()); break;
  case OpType::EltwiseBinaryCompositeScalarOp: runPowScalar(op->type_as_EltwiseBinaryCompositeScalarOp()); break;
  case OpType::DumpTensorOp: runDumpTensor(op->type_as_DumpTensorOp()); break;
  case OpType::LoadTensorOp: runLoadTensor(op->type_as_LoadTensorOp()); break;
  // Annotations and region markers hand their operand on (operations/debug/debug.cpp:18-24, 56-68).
  case OpType::AnnotateOp: runAlias(op->type_as_AnnotateOp()->operand(), op->type_as_AnnotateOp()->result()); break;
  case OpType::RegionStartOp: runAlias(op->type_as_RegionStartOp()->operand(), op->type_as_RegionStartOp()->result()); break;
  case OpType::RegionEndOp: runAlias(op->type_as_RegionEndOp()->operand(), op->type_as_RegionEndOp()->result()); break;
  case OpType::BreakpointOp:
    // The reference drops into Python's pdb (debug.cpp:16,26-28); this runtime embeds no interpreter.
    std::fprintf(stderr, "[ttb200] breakpoint op reached (no debugger is attached by this runtime)\n");
    break;
  case OpType::PrintOp: {
    const auto *o = op->type_as_PrintOp();
    std::fprintf(stderr, "%s\n", o->message() ? o->message()->c_str() : "");
    break;
  }
  case OpType::MemorySnapshotOp: runMemorySnapshot(op->type_as_MemorySnapshotOp()); break;
  case OpType::AllReduceAsyncOp: runAllReduceAsync(op->type_as_AllReduceAsyncOp()); break;
  case OpType::PointToPointOp: runPointToPoint(op->type_as_PointToPointOp()); break;
  case OpType::PrepareConvTranspose2dWeightsOp: {
    const auto *o = op->type_as_PrepareConvTranspose2dWeightsOp();
    runPrepareConv2d(o->weight_tensor(), o->out());
    break;
  }
  case OpType::PrepareConvTranspose2dBiasOp: {
    const auto *o = op->type_as_PrepareConvTranspose2dBiasOp();
    runPrepareConv2d(o->bias_tensor(), o->out());
    break;
  }
  case OpType::NLPCreateQKVHeadsDecodeOp: runNlpCreateQkvHeadsDecode(op->type_as_NLPCreateQKVHeadsDecodeOp()); break;
  case OpType::NLPConcatHeadsDecodeOp: runNlpConcatHeadsDecode(op->type_as_NLPConcatHeadsDecodeOp()); break;
  case OpType::RotaryEmbeddingLlamaOp: runRotaryEmbeddingLlama(op->type_as_RotaryEmbeddingLlamaOp()); break;
  case OpType::MaxPool2dWithIndicesOp: runMaxPool2dWithIndices(op->type_as_MaxPool2dWithIndicesOp()); break;
  case OpType::DropoutOp: runDropout(op->type_as_DropoutOp()); break;
  case OpType::RandOp: runRand(op->type_as_RandOp()); break;
  case OpType::BatchNormTrainingOp: runBatchNormTraining(op->type_as_BatchNormTrainingOp()); break;
  case OpType::GroupNormOp: runGroupNorm(op->type_as_GroupNormOp()); break;
  case OpType::ConvTranspose2dOp: runConvTranspose2d(op->type_as_ConvTranspose2dOp()); break;
  case OpType::Conv1dOp: runConv1d(op->type_as_Conv1dOp()); break;
  case OpType::BitcastConvertOp: runBitcastConvert(op->type_as_BitcastConvertOp()); break;
  case OpType::NLPConcatHeadsOp: runNlpConcatHeads(op->type_as_NLPConcatHeadsOp()); break;
  case OpType::ReductionProdOp: runReductionProd(op->type_as_ReductionProdOp()); break;
  case OpType::BatchNormInferenceOp: runBatchNormInference(op->type_as_BatchNormInferenceOp()); break;
  case OpType::UpsampleOp: runUpsample(op->type_as_UpsampleOp()); break;
  case OpType::PrepareConv2dWeightsOp: {
    const auto *o = op->type_as_PrepareConv2dWeightsOp();
    runPrepareConv2d(o->weight_tensor(), o->out());
    break;
  }
  case OpType::PrepareConv2dBiasOp: {
    const auto *o = op->type_as_PrepareConv2dBiasOp();
    runPrepareConv2d(o->bias_tensor(), o->out());
    break;
  }
  case OpType::EmbeddingOp: runEmbedding(op->type_as_EmbeddingOp()); break;
  case OpType::GatherOp: runGather(op->type_as_GatherOp()); break;
  case OpType::ScatterOp: runScatter(op->type_as_ScatterOp()); break;
  case OpType::SortOp: runSort(op->type_as_SortOp()); break;
  case OpType::TopKOp: runTopK(op->type_as_TopKOp()); break;
  case OpType::SamplingOp: runSampling(op->type_as_SamplingOp()); break;
  case OpType::PagedUpdateCacheOp: runPagedUpdateCache(op->type_as_PagedUpdateCacheOp()); break;
  case OpType::PagedFillCacheOp: runPagedFillCache(op->type_as_PagedFillCacheOp()); break;
  case OpType::PagedScaledDotProductAttentionDecodeOp:
    runPagedSdpaDecode(op->type_as_PagedScaledDotProductAttentionDecodeOp());
    break;
  case OpType::Pool2dOp: runPool2d(op->type_as_Pool2dOp()); break;
  case OpType::GlobalAvgPool2dOp: runGlobalAvgPool2d(op->type_as_GlobalAvgPool2dOp()); break;
  case OpType::PadOp: runPad(op->type_as_PadOp()); break;
  case OpType::FillCacheOp: runFillCache(op->type_as_FillCacheOp()); break;
  case OpType::UpdateCacheOp: runUpdateCache(op->type_as_UpdateCacheOp()); break;
  case OpType::ScaledDotProductAttentionDecodeOp: runSdpaDecode(op->type_as_ScaledDotProductAttentionDecodeOp()); break;
  case OpType::LoadCachedOp: runLoadCached(op->type_as_LoadCachedOp()); break;
  case OpType::FuncCallOp: runFuncCall(op->type_as_FuncCallOp()); break;
  case OpType::BeginTraceCaptureOp: runBeginTraceCapture(op->type_as_BeginTraceCaptureOp()); break;
  case OpType::EndTraceCaptureOp: runEndTraceCapture(op->type_as_EndTraceCaptureOp()); break;
  case OpType::ExecuteTraceOp: runExecuteTrace(op->type_as_ExecuteTraceOp()); break;
  case OpType::CaptureOrExecuteTraceOp: runCaptureOrExecuteTrace(op->type_as_CaptureOrExecuteTraceOp()); break;
  case OpType::WriteTensorOp: runWriteTensor(op->type_as_WriteTensorOp()); break;
  case OpType::CopyOp: runCopy(op->type_as_CopyOp()); break;
  case OpType::CpuOp:
    TTRT_FATAL("CpuOp '", op->type_as_CpuOp()->func_name() ? op->type_as_CpuOp()->func_name()->str() : "",
               "': CPU-hoisted functions are not executed by this target (no CPU fallback); recompile the graph "
               "without CPU hoisting");
  default:
    TTRT_FATAL("unsupported operation ", fbt::EnumNameOpType(op->type_type()));
  }
  return 1;
}

// ---- layout / lifetime ops ----------------------------------------------------------------------
void Executor::runGetDevice(const fbt::GetDeviceOp *op) {
  if (const auto *m = op->mesh()) {
    uint32_t vol = static_cast<uint32_t>(std::max(m->y(), 1) * std::max(m->x(), 1));
    TTRT_ASSERT(vol == dev->worldSize || vol == 1, "GetDeviceOp asks for a ", m->y(), "x", m->x(), " mesh, device has ",
                dev->worldSize, " chips");
  }
}

void Executor::runToDevice(const fbt::ToDeviceOp *op) {
  TensorPtr in = get(op->in());
  if (in->storage == Storage::Host) refuseWhileRecording("a host-to-device copy");
  TensorPtr out = in->storage == Storage::Host ? toDevice(in, dev, in->dtype) : in;
  put(op->out(), out);
}

void Executor::runFromDevice(const fbt::FromDeviceOp *op) {
  TensorPtr in = get(op->in());
  if (in->storage == Storage::Device) refuseWhileRecording("a device-to-host read");
  put(op->out(), in->storage == Storage::Device ? toHostTensor(in, true) : in);
}

void Executor::runToLayout(const fbt::ToLayoutOp *op) {
  TensorPtr in = get(op->in());
  DataType dt = op->dtype().value_or(in->dtype);
  TensorPtr out = in;
  if (in->storage == Storage::Host && refOnDevice(op->out())) {
    out = toDevice(in, dev, dt);
  } else if (in->storage == Storage::Device && dt != in->dtype) {
    out = castOnDevice(in, dt);
  } else if (in->storage == Storage::Device && !refOnDevice(op->out())) {
    out = toHostTensor(in, true);
  }
  if (out == in) {
    // Tilize / untilize only: new handle, same memory.
    auto alias = std::make_shared<TensorImpl>();
    alias->shape = in->shape;
    alias->stride = in->stride;
    alias->dtype = in->dtype;
    alias->storage = in->storage;
    alias->shards = in->shards;
    alias->device = in->device;
    out = alias;
  }
  out->layout = op->layout();
  put(op->out(), out);
}

void Executor::runToMemoryConfig(const fbt::ToMemoryConfigOp *op) {
  // DRAM / L1 / sharding choices have no meaning in HBM: the output aliases the input.
  put(op->out(), get(op->in0()));
}

void Executor::runTypecast(const fbt::TypecastOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = castOnDevice(in, op->dtype());
  if (out == in) {
    auto alias = std::make_shared<TensorImpl>();
    alias->shape = in->shape;
    alias->stride = in->stride;
    alias->dtype = in->dtype;
    alias->storage = in->storage;
    alias->layout = in->layout;
    alias->shards = in->shards;
    alias->device = in->device;
    out = alias;
  }
  put(op->out(), out);
}

void Executor::runDeallocate(const fbt::DeallocateOp *op) {
  TTRT_ASSERT(op->in() != nullptr, "DeallocateOp without operand");
  lazy.erase(op->in()->global_id());
  auto it = pool.find(op->in()->global_id());
  if (it == pool.end()) {
    return;
  }
  // Retained tensors survive program deallocations (reference: operations/deletion/deallocate.cpp).
  if (!it->second->retain || op->force()) {
    pool.erase(it);
  }
}

// ---- creation ops -------------------------------------------------------------------------------
void Executor::runFull(const fbt::FullOp *op) {
  TensorPtr out = allocOut(op->out());
  double v = numberValue(op->fill_value_type(), op->fill_value());
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_fill(out->shards[i]->ptr, ttbDtype(out->dtype), out->volume(), v, r.stream));
  });
  put(op->out(), out);
}

void Executor::runNamedFull(const fbt::NamedFullOp *op) {
  TensorPtr out = allocOut(op->out());
  double v = op->type() == fbt::NamedFullOpType::Ones ? 1.0 : 0.0;
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_fill(out->shards[i]->ptr, ttbDtype(out->dtype), out->volume(), v, r.stream));
  });
  put(op->out(), out);
}

void Executor::runConstant(const fbt::ConstantOp *op) {
  TTRT_ASSERT(op->input() != nullptr, "ConstantOp without data");
  std::vector<uint32_t> shape = refShape(op->out());
  DataType inDt = op->input_dtype();
  size_t vol = prod(shape, 0, shape.size());
  TTRT_ASSERT(op->input()->size() == vol * dataTypeSize(inDt), "ConstantOp data has ", op->input()->size(),
              " bytes, expected ", vol * dataTypeSize(inDt));
  auto host = std::make_shared<TensorImpl>();
  host->shape = shape;
  host->stride = denseStrides(shape);
  host->dtype = inDt;
  host->storage = Storage::Host;
  auto buf = std::make_shared<Buffer>();
  buf->ptr = const_cast<uint8_t *>(op->input()->data());
  buf->bytes = op->input()->size();
  buf->kind = Buffer::Kind::Borrowed;
  buf->keepAlive = bin.handle;
  host->shards.push_back(buf);
  if (refOnDevice(op->out())) {
    refuseWhileRecording("uploading an embedded constant (hoist it out of the traced function)");
    TensorPtr out = toDevice(host, dev, refDtype(op->out()));
    out->layout = refLayout(op->out());
    put(op->out(), out);
  } else {
    put(op->out(), host);
  }
}

void Executor::runEmpty(const fbt::EmptyOp *op) { put(op->out(), allocOut(op->out())); }

void Executor::runArange(const fbt::ArangeOp *op) {
  TensorPtr out = allocOut(op->out());
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_arange(out->shards[i]->ptr, ttbDtype(out->dtype), out->volume(), op->start(), op->step(), r.stream));
  });
  put(op->out(), out);
}

// ---- elementwise ----------------------------------------------------------------------------------
void Executor::runUnary(const fbt::EltwiseUnaryOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(in->volume() == out->volume(), "unary op changes the element count");
  float param = 0.0f;
  if (const auto *p = op->params_as_EltwiseOpWithFloatParams()) param = p->parameter();
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_eltwise_unary(static_cast<int>(op->type()), in->shards[i]->ptr, ttbDtype(in->dtype),
                               out->shards[i]->ptr, ttbDtype(out->dtype), out->volume(), param, r.stream));
  });
  put(op->out(), out);
}

void Executor::runUnaryComposite(const fbt::EltwiseUnaryCompositeOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  using T = fbt::EltwiseUnaryCompositeOpType;
  switch (op->type()) {
  case T::ClampScalar: {
    const auto *p = op->params_as_ClampScalarOpParams();
    TTRT_ASSERT(p != nullptr, "clamp without bounds");
    float lo = numberValue(p->min_type(), p->min()), hi = numberValue(p->max_type(), p->max());
    TTRT_ASSERT(in->dtype == out->dtype, "clamp changes the data type");
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_clamp(in->shards[i]->ptr, ttbDtype(in->dtype), out->shards[i]->ptr, out->volume(), lo, hi, r.stream));
    });
    break;
  }
  case T::Cbrt:
  case T::Log1p: {
    int code = op->type() == T::Cbrt ? 200 : 201;
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_eltwise_unary(code, in->shards[i]->ptr, ttbDtype(in->dtype), out->shards[i]->ptr,
                                 ttbDtype(out->dtype), out->volume(), 0.0f, r.stream));
    });
    break;
  }
  default:
    TTRT_FATAL("unsupported composite unary op ", static_cast<int>(op->type()));
  }
  put(op->out(), out);
}

// numpy-style broadcast strides of `shape` against `outShape` (right aligned, in elements)
static std::vector<int64_t> broadcastStrides(const std::vector<uint32_t> &shape, const std::vector<uint32_t> &outShape) {
  TTRT_ASSERT(shape.size() <= outShape.size(), "operand rank exceeds result rank");
  std::vector<int64_t> dense = denseStrides(shape);
  std::vector<int64_t> s(outShape.size(), 0);
  size_t off = outShape.size() - shape.size();
  for (size_t i = 0; i < shape.size(); ++i) {
    if (shape[i] == outShape[off + i]) {
      s[off + i] = shape[i] == 1 ? 0 : dense[i];
    } else {
      TTRT_ASSERT(shape[i] == 1, "shapes do not broadcast");
      s[off + i] = 0;
    }
  }
  return s;
}

void Executor::runBinary(int opCode, const fbt::TensorRef *lhsRef, const fbt::TensorRef *rhsRef, const fbt::TensorRef *outRef) {
  TensorPtr a = getDevice(lhsRef), b = getDevice(rhsRef);
  TensorPtr out = allocOut(outRef);
  TTRT_ASSERT(out->shape.size() <= 8, "rank above 8");
  std::vector<int64_t> sa = broadcastStrides(a->shape, out->shape), sb = broadcastStrides(b->shape, out->shape);
  std::vector<int64_t> shape(out->shape.begin(), out->shape.end());
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_eltwise_binary(opCode, a->shards[i]->ptr, ttbDtype(a->dtype), b->shards[i]->ptr, ttbDtype(b->dtype),
                                out->shards[i]->ptr, ttbDtype(out->dtype), static_cast<int>(shape.size()), shape.data(),
                                sa.data(), sb.data(), r.stream));
  });
  put(outRef, out);
}

void Executor::runWhere(const fbt::EltwiseTernaryWhereOp *op) {
  TensorPtr c = getDevice(op->first()), a = getDevice(op->second()), b = getDevice(op->third());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(a->dtype == b->dtype && a->dtype == out->dtype, "where branches must share the result type");
  std::vector<int64_t> sc = broadcastStrides(c->shape, out->shape), sa = broadcastStrides(a->shape, out->shape),
                       sb = broadcastStrides(b->shape, out->shape);
  std::vector<int64_t> shape(out->shape.begin(), out->shape.end());
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_where(c->shards[i]->ptr, ttbDtype(c->dtype), a->shards[i]->ptr, b->shards[i]->ptr, ttbDtype(a->dtype),
                       out->shards[i]->ptr, static_cast<int>(shape.size()), shape.data(), sc.data(), sa.data(),
                       sb.data(), r.stream));
  });
  put(op->out(), out);
}

// ---- quantization -----------------------------------------------------------------------------------
namespace {
struct QParams {
  bool perAxis = false;
  float scale = 1.0f;
  int32_t zp = 0;
  const fbt::TensorRef *scaleRef = nullptr;
  const fbt::TensorRef *zpRef = nullptr;
};

QParams readQParams(fbt::QuantizationScale sTy, const void *s, fbt::QuantizationZeroPoint zTy, const void *z) {
  QParams q;
  if (sTy == fbt::QuantizationScale::PerTensorScale) {
    q.scale = static_cast<const fbt::PerTensorScale *>(s)->scale();
  } else if (sTy == fbt::QuantizationScale::PerAxisScale) {
    q.perAxis = true;
    q.scaleRef = static_cast<const fbt::PerAxisScale *>(s)->scale();
  } else {
    TTRT_FATAL("quantization op without a scale");
  }
  if (zTy == fbt::QuantizationZeroPoint::PerTensorZeroPoint) {
    q.zp = static_cast<const fbt::PerTensorZeroPoint *>(z)->zero_point();
  } else if (zTy == fbt::QuantizationZeroPoint::PerAxisZeroPoint) {
    q.zpRef = static_cast<const fbt::PerAxisZeroPoint *>(z)->zero_point();
  }
  return q;
}

// Quantized values live in 32-bit containers when the compiler's default storage width is
// used (lib/Dialect/TTNN/Pipelines/TTNNPipelines.cpp:349-351); this target then clamps to the
// int8 range, which is what the graph's !quant.uniform<i8:...> type means.  Set
// TTB_QUANT_I32_FULL_RANGE=1 for graphs whose quantized type really is 32 bit wide.
int clampI8ForContainer() {
  static const int v = [] {
    const char *e = std::getenv("TTB_QUANT_I32_FULL_RANGE");
    return (e && e[0] == '1') ? 0 : 1;
  }();
  return v;
}
} // namespace

void Executor::runQuantization(const fbt::EltwiseQuantizationOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(in->volume() == out->volume(), "quantization op changes the element count");
  size_t n = out->volume();
  int clampI8 = clampI8ForContainer();
  using T = fbt::EltwiseQuantizationOpType;
  size_t rank = in->shape.size();
  auto axisSplit = [&](size_t &outer, size_t &len, size_t &inner) {
    TTRT_ASSERT(op->axis().has_value(), "per-axis quantization without axis");
    int ax = normDim(*op->axis(), rank);
    outer = prod(in->shape, 0, ax);
    len = in->shape[ax];
    inner = prod(in->shape, ax + 1, rank);
  };
  auto f32Param = [&](const fbt::TensorRef *ref, size_t len) {
    TensorPtr t = castOnDevice(getDevice(ref), DataType::Float32);
    TTRT_ASSERT(t->volume() == len, "per-axis scale has ", t->volume(), " entries, axis has ", len);
    return t;
  };
  auto i32Param = [&](const fbt::TensorRef *ref, size_t len) -> TensorPtr {
    if (!ref) return nullptr;
    TensorPtr t = castOnDevice(getDevice(ref), DataType::Int32);
    TTRT_ASSERT(t->volume() == len, "per-axis zero point has ", t->volume(), " entries, axis has ", len);
    return t;
  };
  if (op->type() == T::Requantize) {
    const auto *p = op->params_as_RequantizeOpParams();
    TTRT_ASSERT(p != nullptr, "requantize without parameters");
    QParams qi = readQParams(p->in_scale_type(), p->in_scale(), p->in_zero_point_type(), p->in_zero_point());
    QParams qo = readQParams(p->out_scale_type(), p->out_scale(), p->out_zero_point_type(), p->out_zero_point());
    if (!qi.perAxis && !qo.perAxis) {
      eachRank([&](size_t i, const RankCtx &r) {
        TTB_CALL(ttb_requantize(in->shards[i]->ptr, ttbDtype(in->dtype), out->shards[i]->ptr, ttbDtype(out->dtype), n,
                                qi.scale, qi.zp, qo.scale, qo.zp, clampI8, r.stream));
      });
    } else {
      TTRT_ASSERT(qi.perAxis && qo.perAxis, "requantize must be per-axis on both sides or on neither");
      size_t outer, len, inner;
      axisSplit(outer, len, inner);
      TensorPtr si = f32Param(qi.scaleRef, len), so = f32Param(qo.scaleRef, len);
      TensorPtr zi = i32Param(qi.zpRef, len), zo = i32Param(qo.zpRef, len);
      eachRank([&](size_t i, const RankCtx &r) {
        TTB_CALL(ttb_requantize_per_axis(in->shards[i]->ptr, ttbDtype(in->dtype), out->shards[i]->ptr,
                                         ttbDtype(out->dtype), outer, len, inner,
                                         static_cast<const float *>(si->shards[i]->ptr),
                                         zi ? static_cast<const int32_t *>(zi->shards[i]->ptr) : nullptr,
                                         static_cast<const float *>(so->shards[i]->ptr),
                                         zo ? static_cast<const int32_t *>(zo->shards[i]->ptr) : nullptr, clampI8,
                                         r.stream));
      });
    }
  } else {
    const auto *p = op->params_as_QuantizeDequantizeOpParams();
    TTRT_ASSERT(p != nullptr, "quantize/dequantize without parameters");
    QParams q = readQParams(p->scale_type(), p->scale(), p->zero_point_type(), p->zero_point());
    bool isQ = op->type() == T::Quantize;
    if (!q.perAxis) {
      eachRank([&](size_t i, const RankCtx &r) {
        if (isQ) {
          TTB_CALL(ttb_quantize(in->shards[i]->ptr, ttbDtype(in->dtype), out->shards[i]->ptr, ttbDtype(out->dtype), n,
                                q.scale, q.zp, clampI8, r.stream));
        } else {
          TTB_CALL(ttb_dequantize(in->shards[i]->ptr, ttbDtype(in->dtype), out->shards[i]->ptr, ttbDtype(out->dtype), n,
                                  q.scale, q.zp, r.stream));
        }
      });
    } else {
      size_t outer, len, inner;
      axisSplit(outer, len, inner);
      TensorPtr s = f32Param(q.scaleRef, len);
      TensorPtr z = i32Param(q.zpRef, len);
      eachRank([&](size_t i, const RankCtx &r) {
        const float *sp = static_cast<const float *>(s->shards[i]->ptr);
        const int32_t *zp = z ? static_cast<const int32_t *>(z->shards[i]->ptr) : nullptr;
        if (isQ) {
          TTB_CALL(ttb_quantize_per_axis(in->shards[i]->ptr, ttbDtype(in->dtype), out->shards[i]->ptr,
                                         ttbDtype(out->dtype), outer, len, inner, sp, zp, clampI8, r.stream));
        } else {
          TTB_CALL(ttb_dequantize_per_axis(in->shards[i]->ptr, ttbDtype(in->dtype), out->shards[i]->ptr,
                                           ttbDtype(out->dtype), outer, len, inner, sp, zp, r.stream));
        }
      });
    }
  }
  put(op->out(), out);
}

// quantize -> requantize -> dequantize with per-tensor parameters and matching scales.
size_t Executor::tryQuantChain(size_t i) {
  const auto *ops = prog->operations();
  using T = fbt::EltwiseQuantizationOpType;
  const auto *q = ops->Get(static_cast<uint32_t>(i))->type_as_EltwiseQuantizationOp();
  if (q->type() != T::Quantize) return 0;
  std::vector<const fbt::Operation *> deallocs;
  size_t j = i + 1;
  const auto *op2 = peek(j, deallocs);
  if (!op2 || op2->type_type() != OpType::EltwiseQuantizationOp) return 0;
  const auto *rq = op2->type_as_EltwiseQuantizationOp();
  if (rq->type() != T::Requantize || rq->in()->global_id() != q->out()->global_id()) return 0;
  size_t k = j + 1;
  const auto *op3 = peek(k, deallocs);
  if (!op3 || op3->type_type() != OpType::EltwiseQuantizationOp) return 0;
  const auto *dq = op3->type_as_EltwiseQuantizationOp();
  if (dq->type() != T::Dequantize || dq->in()->global_id() != rq->out()->global_id()) return 0;
  const auto *pq = q->params_as_QuantizeDequantizeOpParams();
  const auto *prq = rq->params_as_RequantizeOpParams();
  const auto *pdq = dq->params_as_QuantizeDequantizeOpParams();
  if (!pq || !prq || !pdq) return 0;
  QParams a = readQParams(pq->scale_type(), pq->scale(), pq->zero_point_type(), pq->zero_point());
  QParams bi = readQParams(prq->in_scale_type(), prq->in_scale(), prq->in_zero_point_type(), prq->in_zero_point());
  QParams bo = readQParams(prq->out_scale_type(), prq->out_scale(), prq->out_zero_point_type(), prq->out_zero_point());
  QParams c = readQParams(pdq->scale_type(), pdq->scale(), pdq->zero_point_type(), pdq->zero_point());
  if (a.perAxis || bi.perAxis || bo.perAxis || c.perAxis) return 0;
  // the chain must be self-consistent, otherwise run the ops as written
  if (a.scale != bi.scale || a.zp != bi.zp || bo.scale != c.scale || bo.zp != c.zp) return 0;
  DataType d1 = refDtype(q->out()), d2 = refDtype(rq->out());
  if (d1 != d2) return 0;
  DataType din = refDtype(q->in()), dout = refDtype(dq->out());
  bool inOk = din == DataType::BFloat16 || din == DataType::Float32;
  bool outOk = dout == DataType::BFloat16 || dout == DataType::Float32;
  bool qOk = d1 == DataType::Int32 || d1 == DataType::Int8 || d1 == DataType::UInt8;
  if (!inOk || !outOk || !qOk) return 0;

  TensorPtr in = getDevice(q->in());
  // Intermediates are materialised only if something else reads them.
  bool keep1 = !singleUse(q->out()), keep2 = !singleUse(rq->out());
  TensorPtr t1 = keep1 ? allocOut(q->out()) : nullptr;
  TensorPtr t2 = keep2 ? allocOut(rq->out()) : nullptr;
  TensorPtr out = allocOut(dq->out());
  size_t n = out->volume();
  TTRT_ASSERT(in->volume() == n, "quantization chain changes the element count");
  int clampI8 = clampI8ForContainer();
  eachRank([&](size_t r_, const RankCtx &r) {
    TTB_CALL(ttb_quant_chain(in->shards[r_]->ptr, ttbDtype(in->dtype), t1 ? t1->shards[r_]->ptr : nullptr, ttbDtype(d1),
                             t2 ? t2->shards[r_]->ptr : nullptr, ttbDtype(d2), out->shards[r_]->ptr,
                             ttbDtype(out->dtype), n, a.scale, a.zp, bo.scale, bo.zp, clampI8, r.stream));
  });
  if (t1) put(q->out(), t1);
  if (t2) put(rq->out(), t2);
  put(dq->out(), out);
  runDeallocs(deallocs);
  return k + 1 - i;
}

// ---- contractions -------------------------------------------------------------------------------------
bool isQuantizedStorage(DataType dt);

void Executor::runGemm(const fbt::TensorRef *aRef, const fbt::TensorRef *bRef, const fbt::TensorRef *biasRef,
                       const fbt::TensorRef *outRef, bool ta, bool tb, int act, int roundSteps,
                       const fbt::TensorRef *extraRef, int extraOp) {
  if (isQuantizedStorage(refDtype(aRef)) && isQuantizedStorage(refDtype(bRef))) {
    TTRT_ASSERT(!biasRef && !extraRef && act == 0 && roundSteps == 0,
                "a matmul on quantized operands takes no bias, activation or fused operand (dequantize first)");
    runIntGemm(aRef, bRef, outRef, ta, tb, nullptr, 0.0f);
    return;
  }
  TensorPtr a = getDevice(aRef), b = getDevice(bRef);
  TensorPtr bias = biasRef ? getDevice(biasRef) : nullptr;
  TensorPtr extra = extraRef ? getDevice(extraRef) : nullptr;
  TTRT_ASSERT(a->dtype == b->dtype, "matmul operands differ in data type: ", dataTypeName(a->dtype), " vs ",
              dataTypeName(b->dtype));
  // 1-D operands follow numpy: a vector lhs is a row, a vector rhs is a column.
  std::vector<uint32_t> as = a->shape, bs = b->shape;
  if (as.size() == 1) as.insert(as.begin(), 1);
  if (bs.size() == 1) bs.push_back(1);
  TTRT_ASSERT(as.size() >= 2 && bs.size() >= 2, "matmul operands need rank >= 1");
  int64_t M = ta ? as[as.size() - 1] : as[as.size() - 2];
  int64_t K = ta ? as[as.size() - 2] : as[as.size() - 1];
  int64_t Kb = tb ? bs[bs.size() - 1] : bs[bs.size() - 2];
  int64_t N = tb ? bs[bs.size() - 2] : bs[bs.size() - 1];
  TTRT_ASSERT(K == Kb, "matmul inner dimensions differ: ", K, " vs ", Kb);
  int64_t aBatch = static_cast<int64_t>(prod(as, 0, as.size() - 2));
  int64_t bBatch = static_cast<int64_t>(prod(bs, 0, bs.size() - 2));
  int64_t batch = std::max(aBatch, bBatch);
  TTRT_ASSERT((aBatch == batch || aBatch == 1) && (bBatch == batch || bBatch == 1), "matmul batch dimensions do not broadcast");
  int64_t aStride = aBatch == 1 ? 0 : M * K, bStride = bBatch == 1 ? 0 : K * N;
  // A broadcast rhs with a batched lhs is one big GEMM over the stacked rows.
  if (bBatch == 1 && aBatch > 1 && !ta) {
    M *= aBatch;
    batch = 1;
    aStride = 0;
  }
  if (batch == 1 && !ta && tb && !bias && !extra && act == 0 && roundSteps == 0 &&
      static_cast<int64_t>(prod(refShape(outRef), 0, refShape(outRef).size())) == M * N) {
    if (TensorPtr pushed = tryGemmPush(a, b, outRef, M, N, K)) {
      put(outRef, pushed);
      return;
    }
  }
  TensorPtr out = allocForAllReduce(outRef);
  if (!out) out = allocOut(outRef);
  TTRT_ASSERT(static_cast<int64_t>(out->volume()) == batch * M * N, "matmul result has ", out->volume(),
              " elements, expected ", batch * M * N);
  if (bias) {
    TTRT_ASSERT(static_cast<int64_t>(bias->volume()) == N, "bias must have N = ", N, " elements, has ", bias->volume());
  }
  if (extra) {
    TTRT_ASSERT(extra->volume() == out->volume() && extra->dtype == out->dtype, "fused epilogue operand must match the result");
  }
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_gemm_fused(a->shards[i]->ptr, b->shards[i]->ptr, bias ? bias->shards[i]->ptr : nullptr, out->shards[i]->ptr,
                            ttbDtype(a->dtype), bias ? ttbDtype(bias->dtype) : 0, ttbDtype(out->dtype), batch, M, N, K, ta,
                            tb, aStride, bStride, act, roundSteps, extra ? extra->shards[i]->ptr : nullptr,
                            extra ? extraOp : TTB_EXTRA_NONE, r.stream));
  });
  put(outRef, out);
}

// Quantized tensors travel as Int8 / UInt8 or, the compiler's default, as Int32 containers that hold
// int8 values (lib/Dialect/TTNN/Pipelines/TTNNPipelines.cpp:349-351).
bool isQuantizedStorage(DataType dt) { return dt == DataType::Int8 || dt == DataType::UInt8 || dt == DataType::Int32; }

// out = a b on quantized operands: exact 32-bit integer accumulation (tcgen05.mma kind::i8 for the
// weight layout, a CUDA-core kernel otherwise).  An Int32 result holds the accumulators; a float result
// is the accumulator times a scale, which is the dequantize op that followed, fused.  Int32 containers
// are narrowed to Int8 first (their values are in the int8 range by construction).
void Executor::runIntGemm(const fbt::TensorRef *aRef, const fbt::TensorRef *bRef, const fbt::TensorRef *outRef, bool ta, bool tb,
                          const TensorPtr &deqScale, float deqScalar, const fbt::TensorRef *biasRef) {
  TensorPtr a = getDevice(aRef), b = getDevice(bRef);
  TensorPtr bias = biasRef ? getDevice(biasRef) : nullptr;
  if (a->dtype == DataType::Int32 || b->dtype == DataType::Int32) {
    // Only safe while Int32 containers are known to hold int8 values (the rule the quantization ops
    // follow here; TTB_QUANT_I32_FULL_RANGE=1 lifts it, and with it this path).
    TTRT_ASSERT(clampI8ForContainer() != 0,
                "matmul on Int32 containers needs their values in the int8 range (unset TTB_QUANT_I32_FULL_RANGE, or use Int8 tensors)");
    if (a->dtype == DataType::Int32) a = castOnDevice(a, DataType::Int8);
    if (b->dtype == DataType::Int32) b = castOnDevice(b, DataType::Int8);
  }
  std::vector<uint32_t> as = a->shape, bs = b->shape;
  if (as.size() == 1) as.insert(as.begin(), 1);
  if (bs.size() == 1) bs.push_back(1);
  TTRT_ASSERT(as.size() >= 2 && bs.size() >= 2, "matmul operands need rank >= 1");
  int64_t M = ta ? as[as.size() - 1] : as[as.size() - 2];
  int64_t K = ta ? as[as.size() - 2] : as[as.size() - 1];
  int64_t Kb = tb ? bs[bs.size() - 1] : bs[bs.size() - 2];
  int64_t N = tb ? bs[bs.size() - 2] : bs[bs.size() - 1];
  TTRT_ASSERT(K == Kb, "matmul inner dimensions differ: ", K, " vs ", Kb);
  int64_t aBatch = static_cast<int64_t>(prod(as, 0, as.size() - 2));
  int64_t bBatch = static_cast<int64_t>(prod(bs, 0, bs.size() - 2));
  int64_t batch = std::max(aBatch, bBatch);
  TTRT_ASSERT((aBatch == batch || aBatch == 1) && (bBatch == batch || bBatch == 1), "matmul batch dimensions do not broadcast");
  int64_t aStride = aBatch == 1 ? 0 : M * K, bStride = bBatch == 1 ? 0 : K * N;
  if (bBatch == 1 && aBatch > 1 && !ta) {
    M *= aBatch;
    batch = 1;
    aStride = 0;
  }
  TensorPtr out = allocOut(outRef);
  TTRT_ASSERT(static_cast<int64_t>(out->volume()) == batch * M * N, "matmul result has ", out->volume(), " elements, expected ",
              batch * M * N);
  TTRT_ASSERT(out->dtype == DataType::Int32 || out->dtype == DataType::Float32 || out->dtype == DataType::BFloat16 ||
                  out->dtype == DataType::Float16,
              "a matmul on quantized operands produces Int32 accumulators (or, with the dequantize fused, a float type), not ",
              dataTypeName(out->dtype));
  if (deqScale) TTRT_ASSERT(static_cast<int64_t>(deqScale->volume()) == N, "per-channel scale must have N = ", N, " entries");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_gemm_i8_bias(a->shards[i]->ptr, b->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(a->dtype), ttbDtype(b->dtype),
                              ttbDtype(out->dtype), batch, M, N, K, ta, tb, aStride, bStride,
                              deqScale ? static_cast<const float *>(deqScale->shards[i]->ptr) : nullptr, deqScalar,
                              bias ? bias->shards[i]->ptr : nullptr, bias ? ttbDtype(bias->dtype) : 0, r.stream));
  });
  put(outRef, out);
}

// matmul on quantized operands -> dequantize (zero point 0; per tensor, or per axis along the result's
// last dimension): one launch whose epilogue multiplies the integer accumulator by the scale.
size_t Executor::tryQuantizedGemm(size_t i) {
  const auto *ops = prog->operations();
  const auto *op = ops->Get(static_cast<uint32_t>(i));
  const fbt::TensorRef *a, *b, *cur;
  bool ta, tb;
  if (op->type_type() == OpType::MatmulOp) {
    const auto *m = op->type_as_MatmulOp();
    if (activationCode(m->activation()) != TTB_ACT_NONE) return 0;
    a = m->a(); b = m->b(); cur = m->out(); ta = m->transpose_a(); tb = m->transpose_b();
  } else {
    const auto *l = op->type_as_LinearOp();
    if (l->bias() || activationCode(l->activation()) != TTB_ACT_NONE) return 0;
    a = l->a(); b = l->b(); cur = l->out(); ta = l->transpose_a(); tb = l->transpose_b();
  }
  if (!isQuantizedStorage(refDtype(a)) || !isQuantizedStorage(refDtype(b)) || refDtype(cur) != DataType::Int32 || !singleUse(cur))
    return 0;
  std::vector<const fbt::Operation *> deallocs;
  size_t j = i + 1;
  const auto *nop = peek(j, deallocs);
  if (!nop || nop->type_type() != OpType::EltwiseQuantizationOp) return 0;
  const auto *dq = nop->type_as_EltwiseQuantizationOp();
  if (dq->type() != fbt::EltwiseQuantizationOpType::Dequantize || dq->in()->global_id() != cur->global_id() ||
      refShape(dq->out()) != refShape(cur))
    return 0;
  DataType odt = refDtype(dq->out());
  if (odt != DataType::Float32 && odt != DataType::BFloat16 && odt != DataType::Float16) return 0;
  const auto *p = dq->params_as_QuantizeDequantizeOpParams();
  if (!p) return 0;
  QParams q = readQParams(p->scale_type(), p->scale(), p->zero_point_type(), p->zero_point());
  TensorPtr scale;
  if (q.perAxis) {
    const size_t rank = refShape(cur).size();
    if (q.zpRef || !dq->axis().has_value() || normDim(*dq->axis(), rank) != static_cast<int>(rank) - 1 || !q.scaleRef ||
        !pool.count(q.scaleRef->global_id()))
      return 0;
    scale = castOnDevice(getDevice(q.scaleRef), DataType::Float32);
  } else if (q.zp != 0) {
    return 0;
  }
  // optional bias: dequantize -> add(row vector of N), the rounding of the dequantized value kept
  const fbt::TensorRef *result = dq->out(), *biasRef = nullptr;
  size_t last = j;
  if (singleUse(result) && odt != DataType::Float32) {
    std::vector<const fbt::Operation *> d2;
    size_t j2 = j + 1;
    const auto *aop = peek(j2, d2);
    if (aop && aop->type_type() == OpType::EltwiseBinaryOp) {
      const auto *add = aop->type_as_EltwiseBinaryOp();
      const fbt::TensorRef *other = nullptr;
      if (add->type() == fbt::EltwiseBinaryOpType::Add) {
        if (add->lhs()->global_id() == result->global_id()) other = add->rhs();
        else if (add->rhs()->global_id() == result->global_id()) other = add->lhs();
      }
      if (other && other->global_id() != result->global_id() && refShape(add->out()) == refShape(result) &&
          refDtype(add->out()) == odt && pool.count(other->global_id())) {
        std::vector<uint32_t> os = refShape(other);
        const int64_t N = refShape(result).empty() ? 1 : refShape(result).back();
        if (!os.empty() && os.back() == N && static_cast<int64_t>(prod(os, 0, os.size())) == N) {
          biasRef = other;
          result = add->out();
          deallocs.insert(deallocs.end(), d2.begin(), d2.end());
          last = j2;
        }
      }
    }
  }
  runIntGemm(a, b, result, ta, tb, scale, q.scale, biasRef);
  runDeallocs(deallocs);
  return last + 1 - i;
}

static int unaryToAct(fbt::EltwiseUnaryOpType t) {
  switch (t) {
  case fbt::EltwiseUnaryOpType::Relu: return TTB_ACT_RELU;
  case fbt::EltwiseUnaryOpType::Silu: return TTB_ACT_SILU;
  case fbt::EltwiseUnaryOpType::Gelu: return TTB_ACT_GELU;
  case fbt::EltwiseUnaryOpType::Sigmoid: return TTB_ACT_SIGMOID;
  default: return TTB_ACT_NONE;
  }
}

// matmul|linear [-> add(row vector)] [-> relu|silu|gelu|sigmoid] [-> add(tensor) | silu(other) * result],
// each intermediate single-use.
size_t Executor::tryGemmEpilogue(size_t i) {
  const auto *ops = prog->operations();
  const auto *op = ops->Get(static_cast<uint32_t>(i));
  const fbt::TensorRef *a, *b, *bias = nullptr, *cur;
  bool ta, tb;
  int act;
  if (op->type_type() == OpType::MatmulOp) {
    const auto *m = op->type_as_MatmulOp();
    a = m->a(); b = m->b(); cur = m->out(); ta = m->transpose_a(); tb = m->transpose_b();
    act = activationCode(m->activation());
  } else {
    const auto *l = op->type_as_LinearOp();
    a = l->a(); b = l->b(); bias = l->bias(); cur = l->out(); ta = l->transpose_a(); tb = l->transpose_b();
    act = activationCode(l->activation());
  }
  if (act != TTB_ACT_NONE) return 0; // already carries its own activation: run as written
  std::vector<const fbt::Operation *> deallocs;
  int roundSteps = 0;
  size_t next = i + 1, consumedUpTo = i;
  DataType outDt = refDtype(cur);
  int64_t N = refShape(cur).empty() ? 1 : refShape(cur).back();

  // optional bias add
  if (!bias && singleUse(cur)) {
    std::vector<const fbt::Operation *> d2;
    size_t j = next;
    const auto *nop = peek(j, d2);
    if (nop && nop->type_type() == OpType::EltwiseBinaryOp) {
      const auto *add = nop->type_as_EltwiseBinaryOp();
      const fbt::TensorRef *other = nullptr;
      if (add->type() == fbt::EltwiseBinaryOpType::Add) {
        if (add->lhs()->global_id() == cur->global_id()) other = add->rhs();
        else if (add->rhs()->global_id() == cur->global_id()) other = add->lhs();
      }
      if (other && other->global_id() != cur->global_id() && refShape(add->out()) == refShape(cur) &&
          refDtype(add->out()) == outDt) {
        std::vector<uint32_t> os = refShape(other);
        int64_t vol = static_cast<int64_t>(prod(os, 0, os.size()));
        if (vol == N && !os.empty() && os.back() == N && pool.count(other->global_id())) {
          bias = other;
          roundSteps |= 1; // the matmul op stored a rounded product before the add read it
          cur = add->out();
          deallocs.insert(deallocs.end(), d2.begin(), d2.end());
          next = j + 1;
          consumedUpTo = j;
        }
      }
    }
  }
  // optional activation
  if (singleUse(cur)) {
    std::vector<const fbt::Operation *> d2;
    size_t j = next;
    const auto *nop = peek(j, d2);
    if (nop && nop->type_type() == OpType::EltwiseUnaryOp) {
      const auto *u = nop->type_as_EltwiseUnaryOp();
      int code = unaryToAct(u->type());
      if (code != TTB_ACT_NONE && u->in()->global_id() == cur->global_id() && refShape(u->out()) == refShape(cur) &&
          refDtype(u->out()) == outDt) {
        act = code;
        roundSteps |= bias ? 2 : 1; // whatever op fed the activation stored a rounded value
        cur = u->out();
        deallocs.insert(deallocs.end(), d2.begin(), d2.end());
        next = j + 1;
        consumedUpTo = j;
      }
    }
  }
  // optional full-size second operand: a residual add, or SwiGLU gating silu(g) * result
  const fbt::TensorRef *extra = nullptr;
  int extraOp = TTB_EXTRA_NONE;
  auto liveSameAsCur = [&](const fbt::TensorRef *t) {
    return t && t->global_id() != cur->global_id() && refShape(t) == refShape(cur) && refDtype(t) == outDt &&
           pool.count(t->global_id()) != 0;
  };
  if (singleUse(cur) && (outDt == DataType::BFloat16 || outDt == DataType::Float16)) {
    std::vector<const fbt::Operation *> d2;
    size_t j = next;
    const auto *nop = peek(j, d2);
    if (nop && nop->type_type() == OpType::EltwiseBinaryOp) {
      const auto *add = nop->type_as_EltwiseBinaryOp();
      const fbt::TensorRef *other = nullptr;
      if (add->type() == fbt::EltwiseBinaryOpType::Add) {
        if (add->lhs()->global_id() == cur->global_id()) other = add->rhs();
        else if (add->rhs()->global_id() == cur->global_id()) other = add->lhs();
      }
      if (liveSameAsCur(other) && refShape(add->out()) == refShape(cur) && refDtype(add->out()) == outDt) {
        extra = other;
        extraOp = TTB_EXTRA_ADD;
        cur = add->out();
        deallocs.insert(deallocs.end(), d2.begin(), d2.end());
        next = j + 1;
        consumedUpTo = j;
      }
    } else if (nop && nop->type_type() == OpType::EltwiseUnaryOp) {
      const auto *u = nop->type_as_EltwiseUnaryOp();
      std::vector<const fbt::Operation *> d3;
      size_t j2 = j + 1;
      const auto *mop = peek(j2, d3);
      if (u->type() == fbt::EltwiseUnaryOpType::Silu && liveSameAsCur(u->in()) && singleUse(u->out()) &&
          refShape(u->out()) == refShape(cur) && refDtype(u->out()) == outDt && mop &&
          mop->type_type() == OpType::EltwiseBinaryOp) {
        const auto *mul = mop->type_as_EltwiseBinaryOp();
        uint32_t l = mul->lhs()->global_id(), r = mul->rhs()->global_id();
        uint32_t sId = u->out()->global_id(), cId = cur->global_id();
        if (mul->type() == fbt::EltwiseBinaryOpType::Multiply && ((l == sId && r == cId) || (l == cId && r == sId)) &&
            refShape(mul->out()) == refShape(cur) && refDtype(mul->out()) == outDt) {
          extra = u->in();
          extraOp = TTB_EXTRA_SILU_MUL;
          cur = mul->out();
          deallocs.insert(deallocs.end(), d2.begin(), d2.end());
          deallocs.insert(deallocs.end(), d3.begin(), d3.end());
          next = j2 + 1;
          consumedUpTo = j2;
        }
      }
    }
  }
  if (consumedUpTo == i) return 0;
  runGemm(a, b, bias, cur, ta, tb, act, roundSteps, extra, extraOp);
  runDeallocs(deallocs);
  return consumedUpTo + 1 - i;
}

// SwiGLU: g = linear(x, Wg); u = linear(x, Wu); h = multiply(silu(g), u) with g, u and silu(g) used
// nowhere else runs as one contraction whose accumulator holds both projections of an output tile
// (ttb_gemm_swiglu): x is read once and the gate projection never reaches HBM.  The ops may come in
// either of the orders (g, u, silu, multiply) or (g, silu, u, multiply), deallocations in between.
// TTB_DISABLE_SWIGLU_GEMM=1 leaves the pattern to the two-launch form.
size_t Executor::trySwiglu(size_t i) {
  static const bool disabled = [] {
    const char *e = std::getenv("TTB_DISABLE_SWIGLU_GEMM");
    return e && e[0] == '1';
  }();
  if (disabled) return 0;
  const auto *ops = prog->operations();
  struct Proj { const fbt::TensorRef *a, *b, *out; };
  auto plain = [&](const fbt::Operation *op, Proj &pr) {
    if (!op) return false;
    if (op->type_type() == OpType::LinearOp) {
      const auto *l = op->type_as_LinearOp();
      if (l->bias() || l->transpose_a() || !l->transpose_b() || activationCode(l->activation()) != TTB_ACT_NONE) return false;
      pr = {l->a(), l->b(), l->out()};
      return true;
    }
    if (op->type_type() == OpType::MatmulOp) {
      const auto *m = op->type_as_MatmulOp();
      if (m->transpose_a() || !m->transpose_b() || activationCode(m->activation()) != TTB_ACT_NONE) return false;
      pr = {m->a(), m->b(), m->out()};
      return true;
    }
    return false;
  };
  Proj gate, up;
  if (!plain(ops->Get(static_cast<uint32_t>(i)), gate) || !singleUse(gate.out)) return 0;
  std::vector<const fbt::Operation *> deallocs;
  size_t j = i + 1;
  const fbt::Operation *op1 = peek(j, deallocs);
  size_t j2 = j + 1;
  const fbt::Operation *op2 = op1 ? peek(j2, deallocs) : nullptr;
  size_t j3 = j2 + 1;
  const fbt::Operation *op3 = op2 ? peek(j3, deallocs) : nullptr;
  if (!op1 || !op2 || !op3) return 0;
  const fbt::EltwiseUnaryOp *silu = nullptr;
  if (plain(op1, up) && op2->type_type() == OpType::EltwiseUnaryOp) silu = op2->type_as_EltwiseUnaryOp();
  else if (op1->type_type() == OpType::EltwiseUnaryOp && plain(op2, up)) silu = op1->type_as_EltwiseUnaryOp();
  else return 0;
  if (op3->type_type() != OpType::EltwiseBinaryOp) return 0;
  const auto *mul = op3->type_as_EltwiseBinaryOp();
  if (silu->type() != fbt::EltwiseUnaryOpType::Silu || silu->in()->global_id() != gate.out->global_id() ||
      !singleUse(silu->out()) || !singleUse(up.out) || up.a->global_id() != gate.a->global_id() ||
      mul->type() != fbt::EltwiseBinaryOpType::Multiply) {
    return 0;
  }
  const uint32_t l = mul->lhs()->global_id(), r = mul->rhs()->global_id(), sId = silu->out()->global_id(), uId = up.out->global_id();
  if (!((l == sId && r == uId) || (l == uId && r == sId))) return 0;
  DataType dt = refDtype(mul->out());
  if ((dt != DataType::BFloat16 && dt != DataType::Float16) || refDtype(gate.out) != dt || refDtype(up.out) != dt ||
      refDtype(silu->out()) != dt) {
    return 0;
  }
  if (refShape(gate.out) != refShape(up.out) || refShape(mul->out()) != refShape(gate.out) ||
      refShape(silu->out()) != refShape(gate.out)) {
    return 0;
  }
  TensorPtr a = getDevice(gate.a), wg = getDevice(gate.b), wu = getDevice(up.b);
  if (a->dtype != dt || wg->dtype != dt || wu->dtype != dt || wg->shape.size() != 2 || wu->shape != wg->shape || a->shape.empty()) return 0;
  const int64_t K = a->shape.back(), N = wg->shape[0], M = static_cast<int64_t>(a->volume()) / std::max<int64_t>(K, 1);
  if (static_cast<int64_t>(wg->shape[1]) != K || K % 8 != 0 || N % 8 != 0) return 0;
  TensorPtr out = allocOut(mul->out());
  if (static_cast<int64_t>(out->volume()) != M * N) return 0;
  eachRank([&](size_t rk, const RankCtx &rc) {
    TTB_CALL(ttb_gemm_swiglu(a->shards[rk]->ptr, wg->shards[rk]->ptr, wu->shards[rk]->ptr, out->shards[rk]->ptr, ttbDtype(dt), M, N,
                             K, rc.stream));
  });
  put(mul->out(), out);
  runDeallocs(deallocs);
  return j3 + 1 - i;
}

// The rotary_embedding op a projection's result runs into through a head split -- reshape to [batch, seq, heads,
// 128], permute to [batch, heads, seq, 128] -- every link of the chain the only use of the one before.
const fbt::RotaryEmbeddingOp *Executor::ropeAfter(const fbt::TensorRef *out) const {
  auto onlyUser = [&](const fbt::TensorRef *r) -> const fbt::Operation * {
    if (!singleUse(r)) return nullptr;
    auto u = info.firstUse.find(r->global_id());
    return u == info.firstUse.end() ? nullptr : prog->operations()->Get(u->second);
  };
  const auto *o1 = onlyUser(out);
  if (!o1 || o1->type_type() != OpType::ReshapeOp) return nullptr;
  const auto *rs = o1->type_as_ReshapeOp();
  if (rs->in()->global_id() != out->global_id()) return nullptr;
  std::vector<uint32_t> split = refShape(rs->out());
  if (split.size() != 4 || split[3] != 128) return nullptr;
  const auto *o2 = onlyUser(rs->out());
  if (!o2 || o2->type_type() != OpType::PermuteOp) return nullptr;
  const auto *pm = o2->type_as_PermuteOp();
  if (!pm->permutation() || pm->permutation()->size() != 4 || pm->permutation()->Get(0) != 0 || pm->permutation()->Get(1) != 2 ||
      pm->permutation()->Get(2) != 1 || pm->permutation()->Get(3) != 3)
    return nullptr;
  const auto *o3 = onlyUser(pm->out());
  if (!o3 || o3->type_type() != OpType::RotaryEmbeddingOp) return nullptr;
  const auto *rope = o3->type_as_RotaryEmbeddingOp();
  if (rope->input()->global_id() != pm->out()->global_id() || rope->token_index().has_value()) return nullptr;
  if (refDtype(rope->out()) != refDtype(out) || refDtype(rope->cos_cache()) != refDtype(out) || refDtype(rope->sin_cache()) != refDtype(out))
    return nullptr;
  return rope;
}

// Two or three consecutive linear / matmul ops on the same activation (q, k, v projections):
// no bias, no activation, weights as [N, K] (transpose_b), 16-bit, rank-2 problem after
// flattening.  They run as one grouped launch.  Ops whose result feeds an elementwise op right
// after the group are left alone (that pattern belongs to the epilogue fusions).
size_t Executor::tryGroupedGemm(size_t i) {
  const auto *ops = prog->operations();
  struct Item { const fbt::TensorRef *a, *b, *out; };
  auto plain = [&](const fbt::Operation *op, Item &it) {
    if (op->type_type() == OpType::LinearOp) {
      const auto *l = op->type_as_LinearOp();
      if (l->bias() || l->transpose_a() || !l->transpose_b() || activationCode(l->activation()) != TTB_ACT_NONE) return false;
      it = {l->a(), l->b(), l->out()};
      return true;
    }
    if (op->type_type() == OpType::MatmulOp) {
      const auto *m = op->type_as_MatmulOp();
      if (m->transpose_a() || !m->transpose_b() || activationCode(m->activation()) != TTB_ACT_NONE) return false;
      it = {m->a(), m->b(), m->out()};
      return true;
    }
    return false;
  };
  std::vector<Item> items;
  std::vector<const fbt::Operation *> deallocs;
  size_t j = i, last = i;
  while (items.size() < 3) {
    std::vector<const fbt::Operation *> d2;
    size_t k = j;
    const auto *op = items.empty() ? ops->Get(static_cast<uint32_t>(i)) : peek(k, d2);
    Item it;
    if (!op || !plain(op, it)) break;
    if (!items.empty()) {
      if (it.a->global_id() != items[0].a->global_id() || refShape(it.b).size() != 2 || refDtype(it.b) != refDtype(items[0].b) ||
          refShape(it.b)[1] != refShape(items[0].b)[1] || refDtype(it.out) != refDtype(items[0].out))
        break;
      // a deallocation of the shared activation between the ops would end its life too early
      bool freesInput = false;
      for (const auto *d : d2) {
        if (d->type_as_DeallocateOp()->in() && d->type_as_DeallocateOp()->in()->global_id() == it.a->global_id()) freesInput = true;
      }
      if (freesInput) break;
      deallocs.insert(deallocs.end(), d2.begin(), d2.end());
    } else if (refShape(it.b).size() != 2) {
      break;
    }
    items.push_back(it);
    last = items.size() == 1 ? i : k;
    j = last + 1;
  }
  // an elementwise consumer right after the group belongs to an epilogue fusion of the last op
  while (items.size() >= 2) {
    std::vector<const fbt::Operation *> d2;
    size_t k = last + 1;
    const auto *nop = peek(k, d2);
    bool eltwise = nop && (nop->type_type() == OpType::EltwiseBinaryOp || nop->type_type() == OpType::EltwiseUnaryOp);
    if (!eltwise) break;
    return 0; // keep it simple: such chains run op by op with their own fusions
  }
  if (items.size() < 2) return 0;
  DataType abDt = refDtype(items[0].b), cDt = refDtype(items[0].out);
  if ((abDt != DataType::BFloat16 && abDt != DataType::Float16) || refDtype(items[0].a) != abDt) return 0;
  TensorPtr a = getDevice(items[0].a);
  std::vector<uint32_t> as = a->shape;
  if (as.size() < 2) return 0;
  int64_t K = as.back(), M = static_cast<int64_t>(a->volume()) / std::max<int64_t>(K, 1);
  std::vector<TensorPtr> bs, outs;
  std::vector<int64_t> ns;
  for (const Item &it : items) {
    TensorPtr b = getDevice(it.b);
    if (b->shape.size() != 2 || b->shape[1] != K) return 0;
    TensorPtr out = allocOut(it.out);
    if (static_cast<int64_t>(out->volume()) != M * b->shape[0]) return 0;
    bs.push_back(b);
    outs.push_back(out);
    ns.push_back(b->shape[0]);
  }
  // Projections whose result runs into a rotary embedding (through a head split) leave the kernel rotated: the
  // embedding op then has nothing left to do.  One table pair per launch; positions are rows mod seq.
  int ropeMask = 0;
  const fbt::RotaryEmbeddingOp *ropes[3] = {nullptr, nullptr, nullptr};
  TensorPtr cosT, sinT;
  int64_t ropeSeq = 0;
  if (cDt == abDt) {
    for (size_t q = 0; q < items.size(); ++q) {
      const auto *rope = ropeAfter(items[q].out);
      if (!rope || !pool.count(rope->cos_cache()->global_id()) || !pool.count(rope->sin_cache()->global_id())) continue;
      if (ropeMask && (rope->cos_cache()->global_id() != ropes[__builtin_ctz(ropeMask)]->cos_cache()->global_id() ||
                       rope->sin_cache()->global_id() != ropes[__builtin_ctz(ropeMask)]->sin_cache()->global_id()))
        continue;
      std::vector<uint32_t> xs = refShape(rope->input()); // [batch, heads, seq, 128]
      const int64_t seq = xs[2];
      if (static_cast<int64_t>(xs[0]) * seq != M || static_cast<int64_t>(xs[1]) * 128 != ns[q] || (ropeMask && seq != ropeSeq)) continue;
      TensorPtr ct = getDevice(rope->cos_cache()), st = getDevice(rope->sin_cache());
      if (static_cast<int64_t>(ct->volume()) != seq * 128 || static_cast<int64_t>(st->volume()) != seq * 128) continue;
      cosT = ct;
      sinT = st;
      ropeSeq = seq;
      ropes[q] = rope;
      ropeMask |= 1 << q;
    }
  }
  eachRank([&](size_t r, const RankCtx &rc) {
    const void *bp[3];
    void *cp[3];
    for (size_t q = 0; q < items.size(); ++q) {
      bp[q] = bs[q]->shards[r]->ptr;
      cp[q] = outs[q]->shards[r]->ptr;
    }
    if (ropeMask) {
      int rcode = ttb_gemm_grouped_rope(a->shards[r]->ptr, bp, cp, ns.data(), static_cast<int>(items.size()), ttbDtype(abDt), M, K,
                                        cosT->shards[r]->ptr, sinT->shards[r]->ptr, ropeMask, ropeSeq, 128, rc.stream);
      if (rcode == TTB_OK) return;
      // every rank has the same shapes: the first refusal switches the rotation off for all of them
      TTRT_ASSERT(rcode == TTB_ERR_UNSUPPORTED && r == 0, "ttb_gemm_grouped_rope failed (", rcode, "): ", ttb_last_error());
      ropeMask = 0;
    }
    TTB_CALL(ttb_gemm_grouped(a->shards[r]->ptr, bp, cp, ns.data(), static_cast<int>(items.size()), ttbDtype(abDt), ttbDtype(cDt), M,
                              K, rc.stream));
  });
  for (size_t q = 0; q < items.size(); ++q) {
    put(items[q].out, outs[q]);
    if ((ropeMask >> q) & 1) ropeApplied.insert(ropes[q]->input()->global_id());
  }
  runDeallocs(deallocs);
  return last + 1 - i;
}

void Executor::runConv2d(const fbt::Conv2dOp *op, int act, const fbt::TensorRef *extraRef, int extraOp,
                         const fbt::TensorRef *outRef) {
  if (!outRef) outRef = op->out();
  TensorPtr x = getDevice(op->input()), w = getDevice(op->weight());
  TensorPtr bias = op->bias() ? getDevice(op->bias()) : nullptr;
  if (w->preparedFrom) w = w->preparedFrom;            // prepare_conv2d_weights handed the original on
  if (bias && bias->preparedFrom) bias = bias->preparedFrom;
  TensorPtr extra = extraRef ? getDevice(extraRef) : nullptr;
  TensorPtr out = allocOut(outRef);
  if (extra) TTRT_ASSERT(extra->volume() == out->volume() && extra->dtype == out->dtype, "fused epilogue operand must match the result");
  auto two = [](const fb::Vector<int32_t> *v, const char *what, int &a, int &b) {
    TTRT_ASSERT(v && v->size() == 2, "conv2d ", what, " must have 2 entries");
    a = v->Get(0);
    b = v->Get(1);
  };
  int kh, kw, sh, sw, dh, dw;
  two(op->kernel_size(), "kernel_size", kh, kw);
  two(op->stride(), "stride", sh, sw);
  two(op->dilation(), "dilation", dh, dw);
  int pad[4];
  TTRT_ASSERT(op->padding() && (op->padding()->size() == 2 || op->padding()->size() == 4), "conv2d padding must have 2 or 4 entries");
  if (op->padding()->size() == 2) {
    pad[0] = pad[2] = op->padding()->Get(0);
    pad[1] = pad[3] = op->padding()->Get(1);
  } else {
    for (int i = 0; i < 4; ++i) pad[i] = op->padding()->Get(i); // top, left, bottom, right
  }
  int64_t N = op->batch_size(), H = op->input_height(), W = op->input_width(), C = op->in_channels(), O = op->out_channels();
  TTRT_ASSERT(static_cast<int64_t>(x->volume()) == N * H * W * C, "conv2d input has ", x->volume(), " elements, expected N*H*W*C = ",
              N * H * W * C);
  int groups = static_cast<int>(op->groups());
  if (isQuantizedStorage(x->dtype) && isQuantizedStorage(w->dtype)) {
    // Quantized convolution: exact integer accumulation; the result is the Int32 accumulator, or a float
    // type when the dequantize that follows was fused (see tryQuantizedConv).
    TTRT_ASSERT(!bias && !extra && act == TTB_ACT_NONE, "a convolution on quantized operands takes no bias or activation (dequantize first)");
    if (x->dtype == DataType::Int32 || w->dtype == DataType::Int32) {
      TTRT_ASSERT(clampI8ForContainer() != 0, "conv2d on Int32 containers needs their values in the int8 range");
      if (x->dtype == DataType::Int32) x = castOnDevice(x, DataType::Int8);
      if (w->dtype == DataType::Int32) w = castOnDevice(w, DataType::Int8);
    }
    TTRT_ASSERT(out->dtype == DataType::Int32 || out->dtype == DataType::Float32 || out->dtype == DataType::BFloat16 ||
                    out->dtype == DataType::Float16,
                "a convolution on quantized operands produces Int32 accumulators, not ", dataTypeName(out->dtype));
    if (convDeqScale) TTRT_ASSERT(static_cast<int64_t>(convDeqScale->volume()) == O, "per-channel scale must have O = ", O, " entries");
    size_t wsBytes = ttb_conv2d_workspace_bytes(ttbDtype(x->dtype), N, H, W, C, O, kh, kw, sh, sw, pad, dh, dw, groups);
    TensorPtr ws = wsBytes ? makeDeviceTensor(dev, {static_cast<uint32_t>((wsBytes + 3) / 4)}, DataType::UInt32) : nullptr;
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_conv2d_i8(x->shards[i]->ptr, w->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(x->dtype), ttbDtype(w->dtype),
                             ttbDtype(out->dtype), N, H, W, C, O, kh, kw, sh, sw, pad, dh, dw, groups,
                             convDeqScale ? static_cast<const float *>(convDeqScale->shards[i]->ptr) : nullptr, convDeqScalar,
                             ws ? ws->shards[i]->ptr : nullptr, r.stream));
    });
    put(outRef, out);
    return;
  }
  TTRT_ASSERT(x->dtype == w->dtype && x->dtype == out->dtype, "conv2d tensors must share one data type");
  size_t wsBytes = ttb_conv2d_workspace_bytes(ttbDtype(x->dtype), N, H, W, C, O, kh, kw, sh, sw, pad, dh, dw, groups);
  TensorPtr ws = wsBytes ? makeDeviceTensor(dev, {static_cast<uint32_t>((wsBytes + 3) / 4)}, DataType::UInt32) : nullptr;
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_conv2d_fused(x->shards[i]->ptr, w->shards[i]->ptr, bias ? bias->shards[i]->ptr : nullptr, out->shards[i]->ptr,
                              ttbDtype(x->dtype), bias ? ttbDtype(bias->dtype) : 0, N, H, W, C, O, kh, kw, sh, sw, pad, dh, dw,
                              groups, act, extra ? extra->shards[i]->ptr : nullptr, extra ? extraOp : TTB_EXTRA_NONE,
                              ws ? ws->shards[i]->ptr : nullptr, r.stream));
  });
  put(outRef, out);
}

// conv2d on quantized operands -> dequantize (zero point 0; per tensor, or per axis along the channel
// dimension): one contraction whose epilogue multiplies the integer accumulator by the scale.
size_t Executor::tryQuantizedConv(size_t i) {
  const auto *ops = prog->operations();
  const auto *op = ops->Get(static_cast<uint32_t>(i))->type_as_Conv2dOp();
  const fbt::TensorRef *cur = op->out();
  if (op->bias() || !isQuantizedStorage(refDtype(op->input())) || !isQuantizedStorage(refDtype(op->weight())) ||
      refDtype(cur) != DataType::Int32 || !singleUse(cur))
    return 0;
  std::vector<const fbt::Operation *> deallocs;
  size_t j = i + 1;
  const auto *nop = peek(j, deallocs);
  if (!nop || nop->type_type() != OpType::EltwiseQuantizationOp) return 0;
  const auto *dq = nop->type_as_EltwiseQuantizationOp();
  if (dq->type() != fbt::EltwiseQuantizationOpType::Dequantize || dq->in()->global_id() != cur->global_id() ||
      refShape(dq->out()) != refShape(cur))
    return 0;
  DataType odt = refDtype(dq->out());
  if (odt != DataType::Float32 && odt != DataType::BFloat16 && odt != DataType::Float16) return 0;
  const auto *p = dq->params_as_QuantizeDequantizeOpParams();
  if (!p) return 0;
  QParams q = readQParams(p->scale_type(), p->scale(), p->zero_point_type(), p->zero_point());
  TensorPtr scale;
  if (q.perAxis) {
    const size_t rank = refShape(cur).size();
    if (q.zpRef || !dq->axis().has_value() || normDim(*dq->axis(), rank) != static_cast<int>(rank) - 1 || !q.scaleRef ||
        !pool.count(q.scaleRef->global_id()))
      return 0;
    scale = castOnDevice(getDevice(q.scaleRef), DataType::Float32);
  } else if (q.zp != 0) {
    return 0;
  }
  convDeqScale = scale;
  convDeqScalar = q.scale;
  try {
    runConv2d(op, TTB_ACT_NONE, nullptr, TTB_EXTRA_NONE, dq->out());
  } catch (...) {
    convDeqScale.reset();
    throw;
  }
  convDeqScale.reset();
  runDeallocs(deallocs);
  return j + 1 - i;
}

// pointwise conv2d ; pointwise conv2d (the projection of the residual branch) ; add of the two [-> relu]: the end of a
// bottleneck block.  Both convolutions are plain products over the channel dimension, so they run as one launch with
// two accumulators; each product is rounded with its bias as its own op rounds it, the sum as the add does.
size_t Executor::tryPointwisePair(size_t i) {
  const auto *ops = prog->operations();
  const auto *c1 = ops->Get(static_cast<uint32_t>(i))->type_as_Conv2dOp();
  DataType dt = refDtype(c1->out());
  if (dt != DataType::BFloat16 && dt != DataType::Float16) return 0;
  auto pointwise = [&](const fbt::Conv2dOp *c) {
    auto all = [](const fb::Vector<int32_t> *v, int want) {
      if (!v) return false;
      for (int32_t e : *v) {
        if (e != want) return false;
      }
      return v->size() > 0;
    };
    return all(c->kernel_size(), 1) && all(c->stride(), 1) && all(c->padding(), 0) && c->groups() == 1 &&
           refDtype(c->input()) == dt && refDtype(c->weight()) == dt && refDtype(c->out()) == dt &&
           (!c->bias() || refDtype(c->bias()) == dt) && pool.count(c->input()->global_id()) &&
           pool.count(c->weight()->global_id()) && (!c->bias() || pool.count(c->bias()->global_id()));
  };
  if (!pointwise(c1) || !singleUse(c1->out())) return 0;
  std::vector<const fbt::Operation *> deallocs;
  size_t j = i + 1;
  const auto *op2 = peek(j, deallocs);
  if (!op2 || op2->type_type() != OpType::Conv2dOp) return 0;
  const auto *c2 = op2->type_as_Conv2dOp();
  if (!pointwise(c2) || !singleUse(c2->out()) || refShape(c2->out()) != refShape(c1->out())) return 0;
  if (c1->batch_size() != c2->batch_size() || c1->input_height() != c2->input_height() || c1->input_width() != c2->input_width() ||
      c1->out_channels() != c2->out_channels())
    return 0;
  // (deallocations between the ops run after the launch: an operand of the first convolution may be among them)
  size_t j2 = j + 1;
  const auto *op3 = peek(j2, deallocs);
  if (!op3 || op3->type_type() != OpType::EltwiseBinaryOp) return 0;
  const auto *add = op3->type_as_EltwiseBinaryOp();
  if (add->type() != fbt::EltwiseBinaryOpType::Add) return 0;
  const uint32_t l = add->lhs()->global_id(), r = add->rhs()->global_id(), id1 = c1->out()->global_id(), id2 = c2->out()->global_id();
  if (!((l == id1 && r == id2) || (l == id2 && r == id1))) return 0;
  if (refShape(add->out()) != refShape(c1->out()) || refDtype(add->out()) != dt) return 0;
  const fbt::TensorRef *cur = add->out();
  size_t last = j2;
  int act = TTB_ACT_NONE;
  if (singleUse(cur)) {
    std::vector<const fbt::Operation *> d3;
    size_t j3 = j2 + 1;
    const auto *op4 = peek(j3, d3);
    if (op4 && op4->type_type() == OpType::EltwiseUnaryOp) {
      const auto *u = op4->type_as_EltwiseUnaryOp();
      if (u->type() == fbt::EltwiseUnaryOpType::Relu && u->in()->global_id() == cur->global_id() && refShape(u->out()) == refShape(cur) &&
          refDtype(u->out()) == dt) {
        act = TTB_ACT_RELU;
        cur = u->out();
        last = j3;
        deallocs.insert(deallocs.end(), d3.begin(), d3.end());
      }
    }
  }
  TensorPtr x1 = getDevice(c1->input()), w1 = getDevice(c1->weight()), x2 = getDevice(c2->input()), w2 = getDevice(c2->weight());
  TensorPtr b1 = c1->bias() ? getDevice(c1->bias()) : nullptr, b2 = c2->bias() ? getDevice(c2->bias()) : nullptr;
  const int64_t M = static_cast<int64_t>(c1->batch_size()) * c1->input_height() * c1->input_width(), O = c1->out_channels();
  const int64_t K1 = c1->in_channels(), K2 = c2->in_channels();
  if (static_cast<int64_t>(x1->volume()) != M * K1 || static_cast<int64_t>(x2->volume()) != M * K2 ||
      static_cast<int64_t>(w1->volume()) != O * K1 || static_cast<int64_t>(w2->volume()) != O * K2 ||
      (b1 && static_cast<int64_t>(b1->volume()) != O) || (b2 && static_cast<int64_t>(b2->volume()) != O))
    return 0;
  TensorPtr out = allocOut(cur);
  if (static_cast<int64_t>(out->volume()) != M * O) return 0;
  bool taken = true;
  eachRank([&](size_t rk, const RankCtx &rc) {
    if (!taken) return;
    int rcode = ttb_gemm_dual_add(x1->shards[rk]->ptr, w1->shards[rk]->ptr, b1 ? b1->shards[rk]->ptr : nullptr, x2->shards[rk]->ptr,
                                  w2->shards[rk]->ptr, b2 ? b2->shards[rk]->ptr : nullptr, out->shards[rk]->ptr, ttbDtype(dt),
                                  ttbDtype(dt), M, O, K1, K2, act, rc.stream);
    if (rcode == TTB_ERR_UNSUPPORTED && rk == 0) {
      taken = false; // every rank has the same shapes: the ops run one by one
      return;
    }
    TTRT_ASSERT(rcode == TTB_OK, "ttb_gemm_dual_add failed (", rcode, "): ", ttb_last_error());
  });
  if (!taken) return 0;
  put(cur, out);
  runDeallocs(deallocs);
  return last + 1 - i;
}

// conv2d [-> relu], or conv2d -> add(tensor) [-> relu] (a residual branch), intermediates
// single-use.  relu commutes with the rounding of the op before it, so the fused launch gives
// the same bits as the chain.
size_t Executor::tryConvEpilogue(size_t i) {
  const auto *ops = prog->operations();
  const auto *op = ops->Get(static_cast<uint32_t>(i))->type_as_Conv2dOp();
  const fbt::TensorRef *cur = op->out();
  DataType dt = refDtype(cur);
  if (!singleUse(cur)) return 0;
  if (size_t used = tryPointwisePair(i)) return used;
  std::vector<const fbt::Operation *> deallocs;
  size_t next = i + 1, consumedUpTo = i;
  int act = TTB_ACT_NONE, extraOp = TTB_EXTRA_NONE;
  const fbt::TensorRef *extra = nullptr;
  auto reluOf = [&](const fbt::Operation *nop) -> const fbt::EltwiseUnaryOp * {
    if (!nop || nop->type_type() != OpType::EltwiseUnaryOp) return nullptr;
    const auto *u = nop->type_as_EltwiseUnaryOp();
    if (u->type() != fbt::EltwiseUnaryOpType::Relu || u->in()->global_id() != cur->global_id() ||
        refShape(u->out()) != refShape(cur) || refDtype(u->out()) != dt)
      return nullptr;
    return u;
  };
  {
    std::vector<const fbt::Operation *> d2;
    size_t j = next;
    const auto *nop = peek(j, d2);
    if (const auto *u = reluOf(nop)) {
      act = TTB_ACT_RELU;
      cur = u->out();
      deallocs.insert(deallocs.end(), d2.begin(), d2.end());
      next = j + 1;
      consumedUpTo = j;
    } else if (nop && nop->type_type() == OpType::EltwiseBinaryOp && (dt == DataType::BFloat16 || dt == DataType::Float16)) {
      const auto *add = nop->type_as_EltwiseBinaryOp();
      const fbt::TensorRef *other = nullptr;
      if (add->type() == fbt::EltwiseBinaryOpType::Add) {
        if (add->lhs()->global_id() == cur->global_id()) other = add->rhs();
        else if (add->rhs()->global_id() == cur->global_id()) other = add->lhs();
      }
      if (other && other->global_id() != cur->global_id() && refShape(other) == refShape(cur) && refDtype(other) == dt &&
          pool.count(other->global_id()) && refShape(add->out()) == refShape(cur) && refDtype(add->out()) == dt) {
        extra = other;
        extraOp = TTB_EXTRA_ADD;
        cur = add->out();
        deallocs.insert(deallocs.end(), d2.begin(), d2.end());
        next = j + 1;
        consumedUpTo = j;
        if (singleUse(cur)) {
          std::vector<const fbt::Operation *> d3;
          size_t j2 = next;
          const auto *rop = peek(j2, d3);
          if (const auto *u = reluOf(rop)) {
            extraOp = TTB_EXTRA_ADD_RELU;
            cur = u->out();
            deallocs.insert(deallocs.end(), d3.begin(), d3.end());
            next = j2 + 1;
            consumedUpTo = j2;
          }
        }
      }
    }
  }
  if (consumedUpTo == i) return 0;
  runConv2d(op, act, extra, extraOp, cur);
  runDeallocs(deallocs);
  return consumedUpTo + 1 - i;
}


// ---- normalisation / reduction ----------------------------------------------------------------------------
void Executor::runSoftmax(const fbt::SoftmaxOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  size_t rank = in->shape.size();
  int d = normDim(op->dimension(), rank);
  size_t outer = prod(in->shape, 0, d), len = in->shape[d], inner = prod(in->shape, d + 1, rank);
  TTRT_ASSERT(in->dtype == out->dtype, "softmax changes the data type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_softmax(in->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(in->dtype), outer, len, inner, r.stream));
  });
  put(op->out(), out);
}

void Executor::runRmsNorm(const fbt::RMSNormOp *op) {
  TensorPtr in = getDevice(op->input());
  TensorPtr w = op->weight() ? getDevice(op->weight()) : nullptr;
  TensorPtr b = op->bias() ? getDevice(op->bias()) : nullptr;
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(!in->shape.empty(), "rms_norm of a scalar");
  size_t cols = in->shape.back(), rows = in->volume() / std::max<size_t>(cols, 1);
  // Normalisation over the last dimension (the form the TTNN op takes; weight has `cols` entries).
  if (w) TTRT_ASSERT(w->volume() == cols && w->dtype == in->dtype, "rms_norm weight must match the last dimension and data type");
  if (b) TTRT_ASSERT(b->volume() == cols && b->dtype == in->dtype, "rms_norm bias must match the last dimension and data type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_rms_norm(in->shards[i]->ptr, w ? w->shards[i]->ptr : nullptr, b ? b->shards[i]->ptr : nullptr,
                          out->shards[i]->ptr, ttbDtype(in->dtype), rows, cols, op->epsilon(), r.stream));
  });
  put(op->out(), out);
}

// add(a, b) -> rms_norm(sum): one pass; the sum is also written when something else reads it.
size_t Executor::tryAddRmsNorm(size_t i) {
  const auto *ops = prog->operations();
  const auto *add = ops->Get(static_cast<uint32_t>(i))->type_as_EltwiseBinaryOp();
  if (add->type() != fbt::EltwiseBinaryOpType::Add) return 0;
  if (refShape(add->lhs()) != refShape(add->out()) || refShape(add->rhs()) != refShape(add->out())) return 0;
  DataType dt = refDtype(add->out());
  if (refDtype(add->lhs()) != dt || refDtype(add->rhs()) != dt || (dt != DataType::BFloat16 && dt != DataType::Float32)) return 0;
  std::vector<const fbt::Operation *> deallocs;
  size_t j = i + 1;
  const auto *nop = peek(j, deallocs);
  if (!nop || nop->type_type() != OpType::RMSNormOp) return 0;
  const auto *rn = nop->type_as_RMSNormOp();
  if (rn->input()->global_id() != add->out()->global_id() || rn->bias() || !rn->weight()) return 0;
  if (refDtype(rn->out()) != dt || refDtype(rn->weight()) != dt) return 0;
  TensorPtr a = getDevice(add->lhs()), b = getDevice(add->rhs()), w = getDevice(rn->weight());
  bool keepSum = !singleUse(add->out());
  TensorPtr sum = keepSum ? allocOut(add->out()) : nullptr;
  TensorPtr out = allocOut(rn->out());
  size_t cols = out->shape.back(), rows = out->volume() / std::max<size_t>(cols, 1);
  if (w->volume() != cols) return 0;
  eachRank([&](size_t r_, const RankCtx &r) {
    TTB_CALL(ttb_add_rms_norm(a->shards[r_]->ptr, b->shards[r_]->ptr, w->shards[r_]->ptr, sum ? sum->shards[r_]->ptr : nullptr,
                              out->shards[r_]->ptr, ttbDtype(dt), rows, cols, rn->epsilon(), r.stream));
  });
  if (sum) put(add->out(), sum);
  put(rn->out(), out);
  runDeallocs(deallocs);
  return j + 1 - i;
}

// silu(g) -> multiply(silu, u)
size_t Executor::trySiluMul(size_t i) {
  const auto *ops = prog->operations();
  const auto *u = ops->Get(static_cast<uint32_t>(i))->type_as_EltwiseUnaryOp();
  if (u->type() != fbt::EltwiseUnaryOpType::Silu || !singleUse(u->out())) return 0;
  DataType dt = refDtype(u->out());
  if (refDtype(u->in()) != dt || (dt != DataType::BFloat16 && dt != DataType::Float32 && dt != DataType::Float16)) return 0;
  std::vector<const fbt::Operation *> deallocs;
  size_t j = i + 1;
  const auto *nop = peek(j, deallocs);
  if (!nop || nop->type_type() != OpType::EltwiseBinaryOp) return 0;
  const auto *mul = nop->type_as_EltwiseBinaryOp();
  if (mul->type() != fbt::EltwiseBinaryOpType::Multiply) return 0;
  const fbt::TensorRef *other = nullptr;
  if (mul->lhs()->global_id() == u->out()->global_id()) other = mul->rhs();
  else if (mul->rhs()->global_id() == u->out()->global_id()) other = mul->lhs();
  if (!other || other->global_id() == u->out()->global_id()) return 0;
  if (refShape(other) != refShape(u->out()) || refShape(mul->out()) != refShape(u->out())) return 0;
  if (refDtype(other) != dt || refDtype(mul->out()) != dt) return 0;
  TensorPtr g = getDevice(u->in()), up = getDevice(other);
  TensorPtr out = allocOut(mul->out());
  eachRank([&](size_t r_, const RankCtx &r) {
    TTB_CALL(ttb_silu_mul(g->shards[r_]->ptr, up->shards[r_]->ptr, out->shards[r_]->ptr, ttbDtype(dt), out->volume(), r.stream));
  });
  put(mul->out(), out);
  runDeallocs(deallocs);
  return j + 1 - i;
}

void Executor::runReduction(const fbt::ReductionOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  size_t rank = in->shape.size();
  std::vector<int> dims;
  if (op->dim_arg() && op->dim_arg()->size() > 0) {
    for (int32_t d : *op->dim_arg()) dims.push_back(normDim(d, rank));
  } else {
    for (size_t d = 0; d < rank; ++d) dims.push_back(static_cast<int>(d));
  }
  std::sort(dims.begin(), dims.end());
  dims.erase(std::unique(dims.begin(), dims.end()), dims.end());
  bool contiguous = true;
  for (size_t k = 1; k < dims.size(); ++k) contiguous = contiguous && dims[k] == dims[k - 1] + 1;
  TTRT_ASSERT(in->dtype == out->dtype, "reduction changes the data type");
  int code = static_cast<int>(op->type());
  if (contiguous) {
    size_t outer = prod(in->shape, 0, dims.front()), len = prod(in->shape, dims.front(), dims.back() + 1),
           inner = prod(in->shape, dims.back() + 1, rank);
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_reduce(code, in->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(in->dtype), outer, len, inner, r.stream));
    });
  } else {
    // Scattered dims: reduce one dim at a time, innermost first (mean = sums then one division
    // is not bit-identical to nested means, so mean is applied per dim as torch.mean does over
    // a dim tuple only when contiguous; otherwise reject).
    TTRT_ASSERT(op->type() != fbt::ReductionOpType::Mean, "mean over non-adjacent dimensions is not supported");
    TensorPtr cur = in;
    std::vector<uint32_t> shape = in->shape;
    for (int k = static_cast<int>(dims.size()) - 1; k >= 0; --k) {
      int d = dims[k];
      size_t outer = prod(shape, 0, d), len = shape[d], inner = prod(shape, d + 1, shape.size());
      shape[d] = 1;
      TensorPtr nxt = k == 0 ? out : makeDeviceTensor(dev, shape, in->dtype);
      eachRank([&](size_t i, const RankCtx &r) {
        TTB_CALL(ttb_reduce(code, cur->shards[i]->ptr, nxt->shards[i]->ptr, ttbDtype(in->dtype), outer, len, inner, r.stream));
      });
      cur = nxt;
    }
  }
  put(op->out(), out);
}

// layer_norm over the trailing dimensions the weight covers (the last one without a weight).
void Executor::runLayerNorm(const fbt::LayerNormOp *op) {
  TensorPtr in = getDevice(op->input());
  TensorPtr w = op->weight() ? getDevice(op->weight()) : nullptr;
  TensorPtr b = op->bias() ? getDevice(op->bias()) : nullptr;
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(!in->shape.empty(), "layer_norm of a scalar");
  size_t cols = w ? w->volume() : (b ? b->volume() : in->shape.back());
  TTRT_ASSERT(cols > 0 && in->volume() % cols == 0, "layer_norm weight does not cover whole trailing dimensions");
  size_t rows = in->volume() / cols;
  if (w) TTRT_ASSERT(w->dtype == in->dtype, "layer_norm weight must have the input's data type");
  if (b) TTRT_ASSERT(b->volume() == cols && b->dtype == in->dtype, "layer_norm bias must match the weight and the data type");
  TTRT_ASSERT(out->volume() == in->volume() && out->dtype == in->dtype, "layer_norm changes shape or type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_layer_norm(in->shards[i]->ptr, w ? w->shards[i]->ptr : nullptr, b ? b->shards[i]->ptr : nullptr,
                            out->shards[i]->ptr, ttbDtype(in->dtype), rows, cols, op->epsilon(), r.stream));
  });
  put(op->out(), out);
}

// argmax along one dimension, or over everything when the op names none.  Int32 / UInt32 result.
void Executor::runArgMax(const fbt::ReductionArgMaxOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(out->dtype == DataType::Int32 || out->dtype == DataType::UInt32, "argmax produces 32-bit indices");
  size_t rank = in->shape.size(), outer = 1, len = in->volume(), inner = 1;
  if (op->dim().has_value() && rank > 0) {
    int d = normDim(*op->dim(), rank);
    outer = prod(in->shape, 0, d);
    len = in->shape[d];
    inner = prod(in->shape, d + 1, rank);
  }
  TTRT_ASSERT(out->volume() == outer * inner, "argmax result has ", out->volume(), " elements, expected ", outer * inner);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_argmax(in->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(in->dtype), outer, len, inner, r.stream));
  });
  put(op->out(), out);
}

void Executor::runCumSum(const fbt::CumSumOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(out->dtype == in->dtype && out->volume() == in->volume(), "cumsum with a type change is not supported");
  size_t rank = in->shape.size();
  TTRT_ASSERT(rank > 0, "cumsum of a scalar");
  int d = normDim(op->dim(), rank);
  size_t outer = prod(in->shape, 0, d), len = in->shape[d], inner = prod(in->shape, d + 1, rank);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_cumsum(in->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(in->dtype), outer, len, inner, r.stream));
  });
  put(op->out(), out);
}

void Executor::runCumProd(const fbt::CumProdOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(out->dtype == in->dtype && out->volume() == in->volume(), "cumprod with a type change is not supported");
  size_t rank = in->shape.size();
  TTRT_ASSERT(rank > 0, "cumprod of a scalar");
  int d = normDim(op->dim(), rank);
  size_t outer = prod(in->shape, 0, d), len = in->shape[d], inner = prod(in->shape, d + 1, rank);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_cumprod(in->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(in->dtype), outer, len, inner, r.stream));
  });
  put(op->out(), out);
}

// Product over one dimension, or over all of them when dim_arg is absent (operations/reduction/prod.cpp).
void Executor::runReductionProd(const fbt::ReductionProdOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(out->dtype == in->dtype, "prod with a type change is not supported");
  size_t rank = in->shape.size();
  size_t outer = 1, len = in->volume(), inner = 1;
  if (op->dim_arg().has_value()) {
    TTRT_ASSERT(rank > 0, "prod over a dimension of a scalar");
    int d = normDim(static_cast<int>(*op->dim_arg()), rank);
    outer = prod(in->shape, 0, d);
    len = in->shape[d];
    inner = prod(in->shape, d + 1, rank);
  }
  TTRT_ASSERT(out->volume() == outer * inner, "prod result has ", out->volume(), " elements, expected ", outer * inner);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_prod(in->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(in->dtype), outer, len, inner, r.stream));
  });
  put(op->out(), out);
}

// paged_flash_multi_latent_attention_decode (operations/transformer/paged_flash_multi_latent_attention_decode.cpp;
// golden tools/golden/mapping.py:8275-8365): one query token per user, [1, B, H, D], against a paged latent cache
// [blocks, Hkv, block, D]; values are the first head_dim_v columns of the keys unless a paged value cache is given;
// user u sees keys 0 .. cur_pos[u]; the scale defaults to 1, as in the golden.  The user's pages are gathered into one
// sequence and the multi-latent attention kernel runs with one query row per (user, head).
void Executor::runPagedMlaDecode(const fbt::PagedFlashMultiLatentAttentionDecodeOp *op) {
  TTRT_ASSERT(!op->attention_sink(), "attention sinks are not supported");
  TensorPtr q = getDevice(op->query()), kc = getDevice(op->key()), table = getDevice(op->page_table());
  TensorPtr vc = op->value() ? getDevice(op->value()) : nullptr;
  TensorPtr maskIn = op->attention_mask() ? getDevice(op->attention_mask()) : nullptr;
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(q->shape.size() == 4 && q->shape[0] == 1 && kc->shape.size() == 4 && table->shape.size() == 2,
              "paged MLA decode expects query [1, B, H, D], a cache [blocks, Hkv, block, D] and page_table [B, blocks per user]");
  const int64_t B = q->shape[1], Hq = q->shape[2], D = q->shape[3];
  const int64_t numBlocks = kc->shape[0], Hkv = kc->shape[1], blockSize = kc->shape[2], perUser = table->shape[1];
  const int64_t Dv = op->head_dim_v(), Skv = perUser * blockSize;
  TTRT_ASSERT(kc->shape[3] == D && table->shape[0] == B && Hkv > 0 && Hq % Hkv == 0, "paged MLA decode operands do not fit together");
  TTRT_ASSERT(!vc || (vc->shape.size() == 4 && vc->shape[0] == numBlocks && vc->shape[1] == Hkv && vc->shape[2] == blockSize && vc->shape[3] == Dv),
              "the value cache must be [blocks, Hkv, block, head_dim_v]");
  TTRT_ASSERT(kc->dtype == q->dtype && (!vc || vc->dtype == q->dtype) && out->dtype == q->dtype && (!maskIn || maskIn->dtype == q->dtype) &&
                  out->volume() == static_cast<size_t>(B * Hq * Dv),
              "paged MLA decode tensors must share one data type and the result must be [1, B, H, head_dim_v]");
  TensorPtr tbl = table->dtype == DataType::Int32 || table->dtype == DataType::UInt32 ? table : castOnDevice(table, DataType::Int32);
  TensorPtr k = makeDeviceTensor(dev, {static_cast<uint32_t>(B), static_cast<uint32_t>(Hkv), static_cast<uint32_t>(Skv), static_cast<uint32_t>(D)}, q->dtype);
  TensorPtr v = vc ? makeDeviceTensor(dev, {static_cast<uint32_t>(B), static_cast<uint32_t>(Hkv), static_cast<uint32_t>(Skv), static_cast<uint32_t>(Dv)}, q->dtype)
                   : nullptr;
  TensorPtr mask = maskIn;
  int64_t maskB = 1, maskH = 1;
  TensorPtr pos;
  if (maskIn) {
    TTRT_ASSERT(maskIn->shape.size() == 4 && maskIn->shape[3] == Skv && maskIn->volume() == static_cast<size_t>(maskIn->shape[0]) * maskIn->shape[1] * Skv &&
                    (maskIn->shape[0] == 1 || maskIn->shape[0] == B) && (maskIn->shape[1] == 1 || maskIn->shape[1] == Hq),
                "attention_mask must be [B or 1, H or 1, 1, keys]");
    maskB = maskIn->shape[0];
    maskH = maskIn->shape[1];
  } else if (op->is_causal() && op->cur_pos_tensor()) {
    pos = castOnDevice(getDevice(op->cur_pos_tensor()), DataType::Int32);
    TTRT_ASSERT(pos->volume() == static_cast<size_t>(B), "cur_pos_tensor must have one position per user");
    mask = makeDeviceTensor(dev, {static_cast<uint32_t>(B), 1, 1, static_cast<uint32_t>(Skv)}, q->dtype);
    maskB = B;
  }
  const float scale = op->scale().value_or(1.0f);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_paged_gather(kc->shards[i]->ptr, tbl->shards[i]->ptr, k->shards[i]->ptr, ttbDtype(q->dtype), ttbDtype(tbl->dtype), B, Hkv,
                              blockSize, perUser, D, numBlocks, r.stream));
    if (vc) {
      TTB_CALL(ttb_paged_gather(vc->shards[i]->ptr, tbl->shards[i]->ptr, v->shards[i]->ptr, ttbDtype(q->dtype), ttbDtype(tbl->dtype), B, Hkv,
                                blockSize, perUser, Dv, numBlocks, r.stream));
    }
    if (pos) {
      TTB_CALL(ttb_cur_pos_mask(mask->shards[i]->ptr, static_cast<const int32_t *>(pos->shards[i]->ptr), ttbDtype(q->dtype), B, Skv, r.stream));
    }
    // [1, B, H, D] is [B, H, 1, D] in memory: one query row per (user, head)
    TTB_CALL(ttb_flash_mla_prefill(q->shards[i]->ptr, k->shards[i]->ptr, v ? v->shards[i]->ptr : nullptr, mask ? mask->shards[i]->ptr : nullptr,
                                   out->shards[i]->ptr, ttbDtype(q->dtype), B, Hq, Hkv, 1, Skv, D, Dv, maskB, maskH, 0, scale, r.stream));
  });
  put(op->out(), out);
}

// flash_mla_prefill: attention whose values are the first head_dim_v columns of the keys (the shared latent of
// multi-latent attention) unless a value tensor is given; a mask tensor switches the causal flag off, as in the golden.
void Executor::runFlashMlaPrefill(const fbt::FlashMlaPrefillOp *op) {
  TensorPtr q = getDevice(op->query()), k = getDevice(op->key());
  TensorPtr v = op->value() ? getDevice(op->value()) : nullptr, mask = op->attention_mask() ? getDevice(op->attention_mask()) : nullptr;
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(q->shape.size() == 4 && k->shape.size() == 4 && q->shape[0] == k->shape[0] && q->shape[3] == k->shape[3],
              "flash_mla_prefill expects query [B, H, S, D] and key [B, Hkv, Skv, D]");
  const int64_t B = q->shape[0], Hq = q->shape[1], Sq = q->shape[2], D = q->shape[3], Hkv = k->shape[1], Skv = k->shape[2];
  const int64_t Dv = op->head_dim_v();
  TTRT_ASSERT(Hkv > 0 && Hq % Hkv == 0, "query heads must be a multiple of key heads");
  TTRT_ASSERT(!v || (v->shape.size() == 4 && v->shape[0] == B && v->shape[1] == Hkv && v->shape[2] == Skv && v->shape[3] == Dv),
              "flash_mla_prefill value must be [B, Hkv, Skv, head_dim_v]");
  TTRT_ASSERT(k->dtype == q->dtype && (!v || v->dtype == q->dtype) && out->dtype == q->dtype && (!mask || mask->dtype == q->dtype),
              "flash_mla_prefill tensors must share one data type");
  TTRT_ASSERT(out->volume() == static_cast<size_t>(B * Hq * Sq * Dv), "flash_mla_prefill result must be [B, H, S, head_dim_v]");
  int64_t maskB = 1, maskH = 1;
  if (mask) {
    TTRT_ASSERT(mask->shape.size() == 4 && mask->shape[2] == Sq && mask->shape[3] == Skv && (mask->shape[0] == 1 || mask->shape[0] == B) &&
                    (mask->shape[1] == 1 || mask->shape[1] == Hq),
                "attention_mask must be [B or 1, H or 1, S, Skv]");
    maskB = mask->shape[0];
    maskH = mask->shape[1];
  }
  const float scale = op->scale().value_or(1.0f / std::sqrt(static_cast<float>(D)));
  const int causal = op->is_causal() && !mask ? 1 : 0;
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_flash_mla_prefill(q->shards[i]->ptr, k->shards[i]->ptr, v ? v->shards[i]->ptr : nullptr, mask ? mask->shards[i]->ptr : nullptr,
                                   out->shards[i]->ptr, ttbDtype(q->dtype), B, Hq, Hkv, Sq, Skv, D, Dv, maskB, maskH, causal, scale, r.stream));
  });
  put(op->out(), out);
}

// indexer_score_dsa (operations/transformer/indexer_score_dsa.cpp; golden tools/golden/mapping.py:8695-8742): the
// lightning-indexer scores of DeepSeek sparse attention.  On a mesh every device holds a slice of the query sequence;
// its causal window starts behind the rows of the devices before it along cluster_axis, or before it in row-major
// order over the whole mesh when no axis is named (the reference passes the same choice on as its sequence-shard axes).
void Executor::runIndexerScoreDsa(const fbt::IndexerScoreDsaOp *op) {
  TensorPtr q = getDevice(op->query()), k = getDevice(op->key()), w = getDevice(op->weights());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(q->shape.size() == 4 && k->shape.size() == 4 && w->shape.size() == 4, "indexer_score_dsa expects rank-4 tensors");
  const int64_t B = q->shape[0], H = q->shape[1], Sq = q->shape[2], D = q->shape[3], T = k->shape[2];
  TTRT_ASSERT(k->shape[0] == B && k->shape[1] == 1 && k->shape[3] == D, "indexer_score_dsa key must be [B, 1, T, D]");
  TTRT_ASSERT(w->shape[0] == B && w->shape[1] == H && w->shape[2] == Sq && w->shape[3] == 1, "indexer_score_dsa weights must be [B, Hi, Sq, 1]");
  TTRT_ASSERT(k->dtype == q->dtype && w->dtype == q->dtype && out->dtype == q->dtype, "indexer_score_dsa tensors must share one data type");
  TTRT_ASSERT(out->volume() == static_cast<size_t>(B * Sq * T), "indexer_score_dsa result must be [B, 1, Sq, T]");
  const bool named = op->cluster_axis().has_value();
  TTRT_ASSERT(!named || *op->cluster_axis() < 2, "cluster_axis must be 0 or 1");
  const uint32_t cols = std::max<uint32_t>(dev->meshShape[1], 1);
  eachRank([&](size_t i, const RankCtx &r) {
    const uint32_t before = !named ? r.meshRank : (*op->cluster_axis() == 0 ? r.meshRank / cols : r.meshRank % cols);
    TTB_CALL(ttb_indexer_score_dsa(q->shards[i]->ptr, k->shards[i]->ptr, w->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(q->dtype), B, H, Sq,
                                   T, D, static_cast<int64_t>(op->chunk_start_idx()) + static_cast<int64_t>(before) * Sq, r.stream));
  });
  put(op->out(), out);
}

// chunked_scaled_dot_product_attention (operations/transformer/chunked_scaled_dot_product_attention.cpp; golden
// tools/golden/mapping.py:8847-8912): one chunk of a long prefill.  query [B, H, Sq, D] holds positions
// chunk_start .. chunk_start + Sq - 1; keys and values live in a paged cache [blocks, Hkv, block, D] addressed through
// page_table [B, blocks per user]; row r sees keys 0 .. chunk_start + r.  The pages of every user are gathered into
// one sequence (one pass over K and V, small beside the Sq x Skv products), then the causal kernel runs with the
// chunk's offset.  chunk_start_idx is read on the host: it decides how many key tiles the launch covers.
void Executor::runChunkedSdpa(const fbt::ChunkedScaledDotProductAttentionOp *op) {
  TensorPtr q = getDevice(op->query()), kc = getDevice(op->key()), vc = getDevice(op->value());
  TensorPtr table = getDevice(op->page_table());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(q->shape.size() == 4 && kc->shape.size() == 4 && vc->shape == kc->shape && table->shape.size() == 2,
              "chunked attention expects query [B, H, S, D], caches [blocks, Hkv, block, D] and page_table [B, blocks per user]");
  const int64_t B = q->shape[0], Hq = q->shape[1], Sq = q->shape[2], D = q->shape[3];
  const int64_t numBlocks = kc->shape[0], Hkv = kc->shape[1], blockSize = kc->shape[2], perUser = table->shape[1];
  TTRT_ASSERT(kc->shape[3] == D && table->shape[0] == B && Hkv > 0 && Hq % Hkv == 0, "chunked attention operands do not fit together");
  TTRT_ASSERT(kc->dtype == q->dtype && vc->dtype == q->dtype && out->dtype == q->dtype && out->volume() == q->volume(),
              "chunked attention tensors must share one data type");
  refuseWhileRecording("reading chunk_start_idx");
  TensorPtr startT = get(op->chunk_start_idx());
  TTRT_ASSERT(startT->volume() >= 1 && dataTypeSize(startT->dtype) == 4, "chunk_start_idx must hold one 32-bit integer");
  if (startT->storage == Storage::Device) startT = toHostTensor(startT, true);
  const int64_t start = *static_cast<const int32_t *>(startT->shards[0]->ptr);
  const int64_t Skv = perUser * blockSize;
  TTRT_ASSERT(start >= 0 && start + Sq <= Skv, "the chunk [", start, ", ", start + Sq, ") lies outside the ", Skv, " cached positions");
  TensorPtr tbl = table->dtype == DataType::Int32 || table->dtype == DataType::UInt32 ? table : castOnDevice(table, DataType::Int32);
  // Keys beyond the chunk's last row are never visible: gather and attend to the blocks that are.
  const int64_t usedBlocks = (start + Sq + blockSize - 1) / blockSize, used = usedBlocks * blockSize;
  std::vector<uint32_t> seqShape = {static_cast<uint32_t>(B), static_cast<uint32_t>(Hkv), static_cast<uint32_t>(used), static_cast<uint32_t>(D)};
  TensorPtr k = makeDeviceTensor(dev, seqShape, q->dtype), v = makeDeviceTensor(dev, seqShape, q->dtype);
  // the table is read with its own row length; only the first usedBlocks entries of a row are touched
  TensorPtr tblUsed = perUser == usedBlocks ? tbl : stridedView(tbl, {static_cast<uint32_t>(B), static_cast<uint32_t>(usedBlocks)}, {perUser, 1}, 0, tbl->dtype);
  const float scale = op->scale().value_or(1.0f / std::sqrt(static_cast<float>(D)));
  const size_t wsBytes = ttb_sdpa_causal_offset_workspace_bytes(ttbDtype(q->dtype), Sq, used);
  const bool tensorCore = D == 128 && (q->dtype == DataType::BFloat16 || q->dtype == DataType::Float16);
  // small masks are always provided, so that a build or an environment that keeps the tensor-core kernel out still runs
  TensorPtr ws = (tensorCore && wsBytes > (64u << 20)) ? nullptr : makeDeviceTensor(dev, {static_cast<uint32_t>((wsBytes + 3) / 4)}, DataType::UInt32);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_paged_gather(kc->shards[i]->ptr, tblUsed->shards[i]->ptr, k->shards[i]->ptr, ttbDtype(q->dtype), ttbDtype(tblUsed->dtype), B,
                              Hkv, blockSize, usedBlocks, D, numBlocks, r.stream));
    TTB_CALL(ttb_paged_gather(vc->shards[i]->ptr, tblUsed->shards[i]->ptr, v->shards[i]->ptr, ttbDtype(q->dtype), ttbDtype(tblUsed->dtype), B,
                              Hkv, blockSize, usedBlocks, D, numBlocks, r.stream));
    TTB_CALL(ttb_sdpa_causal_offset(q->shards[i]->ptr, k->shards[i]->ptr, v->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(q->dtype), B, Hq,
                                    Hkv, Sq, used, D, start, scale, ws ? ws->shards[i]->ptr : nullptr, r.stream));
  });
  put(op->out(), out);
}

// conv3d over flattened NDHWC activations.  The weight is either the framework's [O, C/g, kD, kH, kW] (also what a
// prepare_conv3d_weights result carries) or TTNN's prepared matrix [kD*kH*kW*C/g, O].
void Executor::runConv3d(const fbt::Conv3dOp *op) {
  TensorPtr x = getDevice(op->input()), w = getDevice(op->weight());
  TensorPtr bias = op->bias() ? getDevice(op->bias()) : nullptr;
  if (w->preparedFrom) w = w->preparedFrom;
  TensorPtr out = allocOut(op->out());
  auto three = [](const fb::Vector<int32_t> *v, const char *what, int (&r)[3]) {
    TTRT_ASSERT(v && v->size() == 3, "conv3d ", what, " must have 3 entries");
    for (int i = 0; i < 3; ++i) r[i] = v->Get(i);
  };
  int k[3], st[3], pd[3];
  three(op->kernel_size(), "kernel_size", k);
  three(op->stride(), "stride", st);
  three(op->padding(), "padding", pd);
  const int N = static_cast<int>(op->batch_size()), D = static_cast<int>(op->input_depth()), H = static_cast<int>(op->input_height()),
            W = static_cast<int>(op->input_width()), C = static_cast<int>(op->in_channels()), O = static_cast<int>(op->out_channels());
  const int groups = static_cast<int>(op->groups()), cg = C / std::max(groups, 1);
  TTRT_ASSERT(x->volume() == static_cast<size_t>(N) * D * H * W * C, "conv3d input has ", x->volume(), " elements, the op says ", N, "x", D,
              "x", H, "x", W, "x", C);
  TTRT_ASSERT(x->dtype == w->dtype && x->dtype == out->dtype && (!bias || (bias->dtype == x->dtype && bias->volume() == static_cast<size_t>(O))),
              "conv3d tensors must share one data type");
  const std::string mode = op->padding_mode() ? op->padding_mode()->str() : "zeros";
  TTRT_ASSERT(mode == "zeros" || mode == "replicate", "conv3d padding mode ", mode, " is not supported");
  const size_t taps = static_cast<size_t>(k[0]) * k[1] * k[2];
  TTRT_ASSERT(w->volume() == taps * cg * O, "conv3d weight has ", w->volume(), " elements, expected ", taps * cg * O);
  int64_t ws[5];
  if (w->shape.size() == 5) { // [O, C/g, kD, kH, kW]
    ws[0] = static_cast<int64_t>(cg) * taps; ws[1] = static_cast<int64_t>(taps); ws[2] = k[1] * k[2]; ws[3] = k[2]; ws[4] = 1;
  } else {                    // [kD*kH*kW*C/g, O]
    ws[0] = 1; ws[1] = O; ws[2] = static_cast<int64_t>(k[1]) * k[2] * cg * O; ws[3] = static_cast<int64_t>(k[2]) * cg * O; ws[4] = static_cast<int64_t>(cg) * O;
  }
  const int od = (D + 2 * pd[0] - k[0]) / st[0] + 1, oh = (H + 2 * pd[1] - k[1]) / st[1] + 1, ow = (W + 2 * pd[2] - k[2]) / st[2] + 1;
  TTRT_ASSERT(out->volume() == static_cast<size_t>(N) * od * oh * ow * O, "conv3d result has ", out->volume(), " elements, expected ", N, "x",
              od, "x", oh, "x", ow, "x", O);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_conv3d(x->shards[i]->ptr, w->shards[i]->ptr, bias ? bias->shards[i]->ptr : nullptr, out->shards[i]->ptr, ttbDtype(x->dtype), N,
                        D, H, W, C, O, k[0], k[1], k[2], st[0], st[1], st[2], pd[0], pd[1], pd[2], groups, mode == "replicate" ? 1 : 0, ws,
                        r.stream));
  });
  put(op->out(), out);
}

void Executor::runGeluBackward(const fbt::ExperimentalEltwiseBinaryBackwardOp *op) {
  TTRT_ASSERT(op->type() == fbt::ExperimentalEltwiseBinaryBackwardOpType::GeluBW, "unknown backward op");
  TensorPtr grad = getDevice(op->grad()), x = getDevice(op->input());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(grad->volume() == x->volume() && out->volume() == x->volume() && grad->dtype == x->dtype && out->dtype == x->dtype,
              "gelu_bw operands must have one shape and data type");
  const std::string approx = op->approximate() ? op->approximate()->str() : "none";
  TTRT_ASSERT(approx == "none" || approx == "tanh", "gelu_bw approximation ", approx, " is not supported");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_gelu_backward(grad->shards[i]->ptr, x->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(x->dtype), x->volume(),
                               approx == "tanh" ? 1 : 0, r.stream));
  });
  put(op->out(), out);
}

void Executor::runEmbeddingBackward(const fbt::EmbeddingBackwardOp *op) {
  TensorPtr idx = getDevice(op->input()), grad = getDevice(op->in_grad());
  TensorPtr out = allocOut(op->out());
  std::vector<uint32_t> ws = refShape(op->weight()); // only the table's shape matters
  TTRT_ASSERT(ws.size() >= 2, "embedding table needs two dimensions");
  const size_t dim = ws.back(), vocab = ws[ws.size() - 2], rows = idx->volume();
  TTRT_ASSERT(grad->volume() == rows * dim && out->volume() == vocab * dim && out->dtype == grad->dtype,
              "embedding_bw: the gradient must be [indices, ", dim, "] and the result [", vocab, ", ", dim, "]");
  TensorPtr scratch = makeDeviceTensor(dev, {static_cast<uint32_t>(vocab), static_cast<uint32_t>(dim)}, DataType::Float32);
  TTRT_ASSERT(scratch->bytes() >= ttb_embedding_backward_workspace_bytes(vocab, dim), "embedding_bw workspace is too small");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_embedding_backward(idx->shards[i]->ptr, grad->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(idx->dtype), ttbDtype(grad->dtype),
                                    rows, vocab, dim, scratch->shards[i]->ptr, r.stream));
  });
  put(op->out(), out);
}

// adamw updates the parameter and the moments in place (operations/ttml/adamw.cpp); the op has no result.
void Executor::runAdamW(const fbt::AdamWOp *op) {
  TensorPtr p = getDevice(op->param()), g = getDevice(op->grad()), m = getDevice(op->exp_avg()), v = getDevice(op->exp_avg_sq());
  TensorPtr vmax = op->max_exp_avg_sq() ? getDevice(op->max_exp_avg_sq()) : nullptr;
  const size_t n = p->volume();
  TTRT_ASSERT(g->volume() == n && m->volume() == n && v->volume() == n && (!vmax || vmax->volume() == n) && v->dtype == m->dtype &&
                  (!vmax || vmax->dtype == m->dtype),
              "adamw tensors must have the parameter's shape and the moments one data type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_adamw(p->shards[i]->ptr, g->shards[i]->ptr, m->shards[i]->ptr, v->shards[i]->ptr, vmax ? vmax->shards[i]->ptr : nullptr,
                       ttbDtype(p->dtype), ttbDtype(g->dtype), ttbDtype(m->dtype), n, op->lr(), op->beta1(), op->beta2(), op->beta1_pow(),
                       op->beta2_pow(), op->epsilon(), op->weight_decay(), op->stochastic_rounding() ? 1 : 0,
                       static_cast<uint32_t>(curOp) * 2654435761u + r.meshRank, r.stream));
  });
  for (const TensorPtr &t : {p, m, v}) t->version = TensorImpl::nextTensorVersion();
  if (vmax) vmax->version = TensorImpl::nextTensorVersion();
}

// ---- mixture of experts ---------------------------------------------------------------------------
TensorPtr Executor::moeLocalIndex(const TensorPtr &mappingIn, uint32_t &experts, uint32_t &devices) {
  TTRT_ASSERT(mappingIn->shape.size() >= 2, "expert_mapping must be [1, 1, experts, devices]");
  experts = mappingIn->shape[mappingIn->shape.size() - 2];
  devices = mappingIn->shape.back();
  TTRT_ASSERT(mappingIn->volume() == static_cast<size_t>(experts) * devices, "expert_mapping has leading dimensions other than 1");
  TTRT_ASSERT(devices == dev->worldSize || dev->worldSize == 1, "expert_mapping covers ", devices, " devices, the mesh has ", dev->worldSize);
  TensorPtr mapping = castOnDevice(mappingIn, DataType::Int32);
  TensorPtr local = makeDeviceTensor(dev, {experts}, DataType::Int32);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_moe_local_index(static_cast<const int32_t *>(mapping->shards[i]->ptr), static_cast<int32_t *>(local->shards[i]->ptr),
                                 static_cast<int>(experts), static_cast<int>(devices), static_cast<int>(r.meshRank % devices), r.stream));
  });
  return local;
}

// all_to_all_dispatch: every device ends up with the global token grid [1, D*B, S, H] (or [1, B, D*S, H]) holding the
// tokens that selected one of its experts (other rows cleared) and with everybody's expert indices.  The exchange is
// an all-gather of both tensors; the mask is local.
void Executor::runAllToAllDispatch(const fbt::AllToAllDispatchOp *op) {
  TensorPtr x = getDevice(op->input_tensor()), idxIn = getDevice(op->expert_indices());
  uint32_t experts = 0, devices = 0;
  TensorPtr local = moeLocalIndex(getDevice(op->expert_mapping()), experts, devices);
  TensorPtr out = allocOut(op->dispatched()), meta = allocOut(op->metadata());
  const uint32_t n = meshAxisSize(op->cluster_axis());
  const size_t hidden = x->shape.back(), k = idxIn->shape.back();
  const size_t rows = x->volume() / std::max<size_t>(hidden, 1);
  TTRT_ASSERT(idxIn->volume() == rows * k, "expert_indices must have one row of ", k, " experts per token");
  TTRT_ASSERT(out->volume() == x->volume() * n && out->dtype == x->dtype && meta->volume() == idxIn->volume() * n && meta->dtype == idxIn->dtype,
              "all_to_all_dispatch results must hold the tokens and indices of all ", n, " devices");
  // Device-major order is the result itself when the devices' tokens are concatenated along the batch; along the
  // sequence each batch row interleaves the devices.
  TTRT_ASSERT(out->shape.size() == 4 && x->shape.size() == 4, "all_to_all_dispatch expects 4-D tokens");
  const size_t batch = x->shape[0], seq = rows / std::max<size_t>(batch, 1);
  const bool seqConcat = n > 1 && out->shape[1] == batch && out->shape[2] == seq * n && batch > 1;
  TensorPtr stagedX = seqConcat ? makeDeviceTensor(dev, {n, static_cast<uint32_t>(x->volume())}, x->dtype) : out;
  TensorPtr stagedI = seqConcat ? makeDeviceTensor(dev, {n, static_cast<uint32_t>(idxIn->volume())}, idxIn->dtype) : meta;
  if (n > 1) {
    refuseWhileRecording("a collective");
    TTB_CALL(ttb_group_start());
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_all_gather(r.comm, x->shards[i]->ptr, stagedX->shards[i]->ptr, x->volume(), ttbDtype(x->dtype), r.stream));
      TTB_CALL(ttb_all_gather(r.comm, idxIn->shards[i]->ptr, stagedI->shards[i]->ptr, idxIn->volume(), ttbDtype(idxIn->dtype), r.stream));
    });
    TTB_CALL(ttb_group_end());
  } else {
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_memcpy_d2d(out->shards[i]->ptr, x->shards[i]->ptr, x->bytes(), r.stream));
      TTB_CALL(ttb_memcpy_d2d(meta->shards[i]->ptr, idxIn->shards[i]->ptr, idxIn->bytes(), r.stream));
    });
  }
  if (seqConcat) {
    // staged [n, batch, seq, w] -> [batch, n, seq, w]
    auto interleave = [&](const TensorPtr &src, const TensorPtr &dst, size_t width) {
      std::vector<int64_t> shape = {static_cast<int64_t>(batch), static_cast<int64_t>(n), static_cast<int64_t>(seq * width)};
      std::vector<int64_t> strides = {static_cast<int64_t>(seq * width), static_cast<int64_t>(batch * seq * width), 1};
      eachRank([&](size_t i, const RankCtx &r) {
        TTB_CALL(ttb_strided_copy(src->shards[i]->ptr, dst->shards[i]->ptr, static_cast<int>(dataTypeSize(src->dtype)), 3, shape.data(),
                                  strides.data(), 0, r.stream));
      });
    };
    interleave(stagedX, out, hidden);
    interleave(stagedI, meta, k);
  }
  TensorPtr idx32 = castOnDevice(meta, DataType::Int32);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_moe_dispatch_mask(out->shards[i]->ptr, static_cast<const int32_t *>(idx32->shards[i]->ptr),
                                   static_cast<const int32_t *>(local->shards[i]->ptr), ttbDtype(out->dtype), rows * n, hidden,
                                   static_cast<int>(k), static_cast<int>(experts), r.stream));
  });
  put(op->dispatched(), out);
  put(op->metadata(), meta);
}

// all_to_all_dispatch_metadata (operations/ccl/all_to_all_dispatch_metadata.cpp; golden tools/golden/mapping.py:1656-1760):
// per device [1, 1, M, H] tokens with [1, 1, M, K] expert indices and scores; every device gets [1, D*M, H] holding the
// tokens routed to it (zeros elsewhere) and the indices and scores of all devices.  expert_mapping is [.., D, E] with
// entry [d, e] = the mesh coordinate that owns expert e.  The persistent buffers and the semaphore of the Tensix
// implementation are not used.
void Executor::runAllToAllDispatchMetadata(const fbt::AllToAllDispatchMetadataOp *op) {
  TensorPtr x = getDevice(op->input_tensor()), idxIn = getDevice(op->expert_indices()), scrIn = getDevice(op->expert_scores());
  TensorPtr owner = castOnDevice(getDevice(op->expert_mapping()), DataType::Int32);
  TTRT_ASSERT(!owner->shape.empty(), "expert_mapping must be [devices, experts]");
  const uint32_t experts = owner->shape.back();
  TensorPtr local = makeDeviceTensor(dev, {experts}, DataType::Int32);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_moe_local_index_owner(static_cast<const int32_t *>(owner->shards[i]->ptr), static_cast<int32_t *>(local->shards[i]->ptr),
                                       static_cast<int>(experts), static_cast<int>(r.meshRank), r.stream));
  });
  TensorPtr out = allocOut(op->dispatched()), idxOut = allocOut(op->indices()), scrOut = allocOut(op->scores());
  const uint32_t n = meshAxisSize(op->cluster_axis());
  const size_t hidden = x->shape.back(), k = idxIn->shape.back(), rows = x->volume() / std::max<size_t>(hidden, 1);
  TTRT_ASSERT(idxIn->volume() == rows * k && scrIn->volume() == rows * k, "expert_indices / expert_scores must be [tokens, ", k, "]");
  TTRT_ASSERT(out->volume() == x->volume() * n && out->dtype == x->dtype && idxOut->volume() == idxIn->volume() * n &&
                  idxOut->dtype == idxIn->dtype && scrOut->volume() == scrIn->volume() * n && scrOut->dtype == scrIn->dtype,
              "all_to_all_dispatch_metadata results must hold the tokens, indices and scores of all ", n, " devices");
  if (n > 1) {
    refuseWhileRecording("a collective");
    TTB_CALL(ttb_group_start());
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_all_gather(r.comm, x->shards[i]->ptr, out->shards[i]->ptr, x->volume(), ttbDtype(x->dtype), r.stream));
      TTB_CALL(ttb_all_gather(r.comm, idxIn->shards[i]->ptr, idxOut->shards[i]->ptr, idxIn->volume(), ttbDtype(idxIn->dtype), r.stream));
      TTB_CALL(ttb_all_gather(r.comm, scrIn->shards[i]->ptr, scrOut->shards[i]->ptr, scrIn->volume(), ttbDtype(scrIn->dtype), r.stream));
    });
    TTB_CALL(ttb_group_end());
  } else {
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_memcpy_d2d(out->shards[i]->ptr, x->shards[i]->ptr, x->bytes(), r.stream));
      TTB_CALL(ttb_memcpy_d2d(idxOut->shards[i]->ptr, idxIn->shards[i]->ptr, idxIn->bytes(), r.stream));
      TTB_CALL(ttb_memcpy_d2d(scrOut->shards[i]->ptr, scrIn->shards[i]->ptr, scrIn->bytes(), r.stream));
    });
  }
  TensorPtr idx32 = castOnDevice(idxOut, DataType::Int32);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_moe_dispatch_mask(out->shards[i]->ptr, static_cast<const int32_t *>(idx32->shards[i]->ptr),
                                   static_cast<const int32_t *>(local->shards[i]->ptr), ttbDtype(out->dtype), rows * n, hidden,
                                   static_cast<int>(k), static_cast<int>(experts), r.stream));
  });
  put(op->dispatched(), out);
  put(op->indices(), idxOut);
  put(op->scores(), scrOut);
}

// topk_router_gpt (operations/reduction/topk_router_gpt.cpp; golden tools/golden/mapping.py:5960-5992): router logits
// = input @ weight (rounded to the input type) + bias (rounded), the k largest per token in descending order, and the
// softmax over those k values.
void Executor::runTopKRouterGpt(const fbt::TopKRouterGptOp *op) {
  TensorPtr x = getDevice(op->input()), w = getDevice(op->weight()), bias = getDevice(op->bias());
  TTRT_ASSERT(x->shape.size() == 2 && w->shape.size() == 2 && w->shape[0] == x->shape[1], "topk_router_gpt expects input [B, H] and weight [H, E]");
  const int64_t B = x->shape[0], H = x->shape[1], E = w->shape[1];
  const size_t k = static_cast<size_t>(op->k());
  TTRT_ASSERT(bias->volume() == static_cast<size_t>(B * E) && bias->dtype == x->dtype && w->dtype == x->dtype,
              "topk_router_gpt bias must be [B, E] in the input's data type");
  TTRT_ASSERT(k >= 1 && static_cast<int64_t>(k) <= E, "k outside [1, experts]");
  TensorPtr logits = makeDeviceTensor(dev, {static_cast<uint32_t>(B), static_cast<uint32_t>(E)}, x->dtype);
  int64_t shape[2] = {B, E}, strides[2] = {E, 1};
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_gemm(x->shards[i]->ptr, w->shards[i]->ptr, nullptr, logits->shards[i]->ptr, ttbDtype(x->dtype), 0, ttbDtype(x->dtype), 1, B, E,
                      H, 0, 0, 0, 0, TTB_ACT_NONE, 1, r.stream));
    TTB_CALL(ttb_eltwise_binary(static_cast<int>(fbt::EltwiseBinaryOpType::Add), logits->shards[i]->ptr, ttbDtype(x->dtype),
                                bias->shards[i]->ptr, ttbDtype(x->dtype), logits->shards[i]->ptr, ttbDtype(x->dtype), 2, shape, strides,
                                strides, r.stream));
  });
  TensorPtr indices = allocOut(op->expert_indices()), weights = allocOut(op->expert_weights());
  TTRT_ASSERT(indices->volume() == static_cast<size_t>(B) * k && weights->volume() == static_cast<size_t>(B) * k,
              "topk_router_gpt results must be [B, k]");
  TensorPtr top = makeDeviceTensor(dev, {static_cast<uint32_t>(B), static_cast<uint32_t>(k)}, x->dtype);
  const size_t wsBytes = ttb_sort_workspace_bytes(static_cast<size_t>(B), static_cast<size_t>(E));
  TensorPtr ws = makeDeviceTensor(dev, {static_cast<uint32_t>((wsBytes + 3) / 4)}, DataType::UInt32);
  TensorPtr soft = weights->dtype == x->dtype ? weights : makeDeviceTensor(dev, top->shape, x->dtype);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_sort(logits->shards[i]->ptr, top->shards[i]->ptr, indices->shards[i]->ptr, ttbDtype(x->dtype), ttbDtype(indices->dtype),
                      static_cast<size_t>(B), static_cast<size_t>(E), k, 1, ws->shards[i]->ptr, wsBytes, r.stream));
    TTB_CALL(ttb_softmax(top->shards[i]->ptr, soft->shards[i]->ptr, ttbDtype(x->dtype), static_cast<size_t>(B), k, 1, r.stream));
  });
  put(op->expert_indices(), indices);
  put(op->expert_weights(), soft == weights ? weights : castOnDevice(soft, weights->dtype));
}

// all_to_all_combine: expert outputs [E_local, global tokens, H] go back to the devices their tokens came from,
// out[slot, b, s, :] = the output of the expert in metadata[token, slot].  Every device writes, for every destination,
// the rows it owns (zeros elsewhere); a sum reduce-scatter delivers them (one owner per row, so the sum is exact).
void Executor::runAllToAllCombine(const fbt::AllToAllCombineOp *op) {
  TensorPtr x = getDevice(op->input_tensor());
  uint32_t experts = 0, devices = 0;
  TensorPtr local = moeLocalIndex(getDevice(op->expert_mapping()), experts, devices);
  TensorPtr meta = castOnDevice(getDevice(op->expert_metadata()), DataType::Int32);
  TensorPtr out = allocOut(op->out());
  const uint32_t n = meshAxisSize(op->cluster_axis());
  TTRT_ASSERT(x->shape.size() == 4 && out->shape.size() == 4 && meta->shape.size() == 4, "all_to_all_combine expects 4-D tensors");
  const uint32_t localExperts = x->shape[0], gBatch = x->shape[1], gSeq = x->shape[2], hidden = x->shape[3];
  const uint32_t k = out->shape[0], batch = out->shape[1], seq = out->shape[2];
  TTRT_ASSERT(k == op->num_experts_per_tok() && meta->shape[3] >= k && meta->shape[1] == gBatch && meta->shape[2] == gSeq,
              "expert_metadata must be [1, ", gBatch, ", ", gSeq, ", >= ", k, "]");
  TTRT_ASSERT(meta->shape[3] == k, "expert_metadata with more slots than num_experts_per_tok is not supported");
  const bool seqSharded = op->output_shard_dim() == 2 && n > 1;
  TTRT_ASSERT(out->shape[3] == hidden && out->dtype == x->dtype &&
                  (seqSharded ? (batch == gBatch && seq * n == gSeq) : (batch * n == gBatch && seq == gSeq)),
              "all_to_all_combine result must be this device's share of the ", gBatch, " x ", gSeq, " tokens");
  TensorPtr partial = n > 1 ? makeDeviceTensor(dev, {n, k, batch, seq, hidden}, x->dtype) : out;
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_moe_combine_partial(x->shards[i]->ptr, static_cast<const int32_t *>(meta->shards[i]->ptr),
                                     static_cast<const int32_t *>(local->shards[i]->ptr), partial->shards[i]->ptr, ttbDtype(x->dtype),
                                     static_cast<int>(n), static_cast<int>(k), static_cast<int>(batch), static_cast<int>(seq), hidden,
                                     static_cast<int>(experts), static_cast<int>(localExperts), seqSharded ? 1 : 0, r.stream));
  });
  if (n > 1) {
    refuseWhileRecording("a collective");
    TTB_CALL(ttb_group_start());
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_reduce_scatter(r.comm, partial->shards[i]->ptr, out->shards[i]->ptr, out->volume(), ttbDtype(x->dtype), 0, r.stream));
    });
    TTB_CALL(ttb_group_end());
  }
  put(op->out(), out);
}

void Executor::runMoeExpertTokenRemap(const fbt::MoeExpertTokenRemapOp *op) {
  TensorPtr topk = getDevice(op->topk_tensor());
  uint32_t experts = 0, devices = 0;
  TensorPtr local = moeLocalIndex(getDevice(op->expert_mapping()), experts, devices);
  TensorPtr meta = castOnDevice(getDevice(op->expert_metadata()), DataType::Int32);
  TensorPtr mapping = allocOut(op->mapping()), reduced = allocOut(op->reduced());
  TTRT_ASSERT(topk->shape.back() == experts, "topk_tensor must have one column per expert (", experts, ")");
  const size_t tokens = topk->volume() / experts, k = meta->shape.back();
  TTRT_ASSERT(meta->volume() == tokens * k, "expert_metadata must have one row per token");
  const uint32_t localExperts = mapping->shape.back(), reduction = op->reduction_size();
  TTRT_ASSERT(reduction > 0 && mapping->volume() == tokens * localExperts && mapping->dtype == topk->dtype &&
                  reduced->volume() == (tokens + reduction - 1) / reduction * localExperts,
              "moe_expert_token_remap results must be [tokens, local experts] and [ceil(tokens / ", reduction, "), local experts]");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_moe_expert_token_remap(topk->shards[i]->ptr, static_cast<const int32_t *>(meta->shards[i]->ptr),
                                        static_cast<const int32_t *>(local->shards[i]->ptr), mapping->shards[i]->ptr, reduced->shards[i]->ptr,
                                        ttbDtype(topk->dtype), ttbDtype(reduced->dtype), tokens, static_cast<int>(k),
                                        static_cast<int>(experts), static_cast<int>(localExperts), static_cast<int>(reduction), r.stream));
  });
  put(op->mapping(), mapping);
  put(op->reduced(), reduced);
}

// sparse_matmul: token blocks against expert weights, only where the sparsity tensor is non-zero.
//   b sparse:    a [A, B, M, K], b [1, E, K, N], sparsity [A, B, 1, E] -> [A, B, 1, E, M, N]
//   a sparse:    a [A, E, M, K], b [1, E, K, N], sparsity [1, 1, A, E] -> [A, E, M, N]
//   both sparse: a [1, E, M, K], b [1, E, K, N], sparsity [1, 1, 1, E] -> [1, E, M, N]
void Executor::runSparseMatmul(const fbt::SparseMatmulOp *op) {
  TensorPtr a = getDevice(op->a()), b = getDevice(op->b()), sp = getDevice(op->sparsity());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(a->shape.size() == 4 && b->shape.size() == 4 && b->shape[0] == 1, "sparse_matmul expects a [.., .., M, K] and b [1, E, K, N]");
  const int64_t E = b->shape[1], K = b->shape[2], N = b->shape[3], M = a->shape[2];
  TTRT_ASSERT(a->shape[3] == K, "inner dimensions differ: ", a->shape[3], " vs ", K);
  const bool aSparse = op->is_input_a_sparse();
  TTRT_ASSERT(aSparse || op->is_input_b_sparse(), "sparse_matmul needs at least one sparse operand");
  int64_t entries;
  if (aSparse) {
    TTRT_ASSERT(a->shape[1] == E, "a must have one block per expert (", E, ")");
    entries = static_cast<int64_t>(a->shape[0]) * E;
  } else {
    entries = static_cast<int64_t>(a->shape[0]) * a->shape[1] * E;
  }
  TTRT_ASSERT(static_cast<int64_t>(sp->volume()) == entries, "the sparsity tensor must have ", entries, " entries");
  TTRT_ASSERT(static_cast<int64_t>(out->volume()) == entries * M * N && out->dtype == a->dtype && b->dtype == a->dtype,
              "sparse_matmul result must be [entries, M, N] in the operands' data type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_sparse_matmul(a->shards[i]->ptr, b->shards[i]->ptr, sp->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(a->dtype),
                               ttbDtype(sp->dtype), entries, E, aSparse ? 1 : 0, M, N, K, r.stream));
  });
  put(op->out(), out);
}

static int fusedActivationCode(const fb::String *s) {
  if (!s || s->size() == 0) return 0;
  std::string name = s->str();
  if (name.size() > 7 && name.compare(name.size() - 7, 7, "_approx") == 0) name.resize(name.size() - 7);
  static const char *names[] = {"", "relu", "relu6", "silu", "mish", "sigmoid", "hardsigmoid", "tanh", "log", "softplus", "gelu", "sqrt"};
  for (int i = 1; i < 12; ++i) {
    if (name == names[i]) return i;
  }
  TTRT_FATAL("unsupported fused activation '", s->str(), "'");
}

// act(rms_norm(input + residual) * weight + bias) in one pass, the sum kept in f32 (tools/golden/mapping.py:1291-1326).
void Executor::runDitRmsNorm(const fbt::DitRMSNormUnaryFusedOp *op) {
  TensorPtr x = getDevice(op->input());
  TensorPtr w = op->weight() ? getDevice(op->weight()) : nullptr, b = op->bias() ? getDevice(op->bias()) : nullptr;
  TensorPtr res = op->residual_input() ? getDevice(op->residual_input()) : nullptr;
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(!x->shape.empty(), "rms norm of a scalar");
  const size_t cols = x->shape.back(), rows = x->volume() / std::max<size_t>(cols, 1);
  TTRT_ASSERT((!w || (w->volume() == cols && w->dtype == x->dtype)) && (!b || (b->volume() == cols && b->dtype == x->dtype)) &&
                  (!res || (res->volume() == x->volume() && res->dtype == x->dtype)) && out->dtype == x->dtype &&
                  out->volume() == x->volume(),
              "dit_rms_norm_unary_fused operands must match the input's last dimension and data type");
  const int act = fusedActivationCode(op->activation());
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_rms_norm_apply(x->shards[i]->ptr, res ? res->shards[i]->ptr : nullptr, w ? w->shards[i]->ptr : nullptr,
                                b ? b->shards[i]->ptr : nullptr, nullptr, out->shards[i]->ptr, ttbDtype(x->dtype), rows, cols, cols,
                                op->epsilon(), act, r.stream));
  });
  put(op->out(), out);
}

// RMS norm of rows whose columns are split over a mesh axis: local sums of squares, one all-reduce of 4 bytes per
// row, local normalisation with the weight slice (tools/golden/mapping.py:1329-1415).  The op's `stats` scratch
// tensor and its semaphore belong to the Tensix implementation and are not touched.
void Executor::runDistributedRmsNorm(const fbt::DistributedRMSNormOp *op) {
  TensorPtr x = getDevice(op->input());
  TensorPtr w = op->weight() ? getDevice(op->weight()) : nullptr, res = op->residual() ? getDevice(op->residual()) : nullptr;
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(!x->shape.empty(), "rms norm of a scalar");
  const size_t cols = x->shape.back(), rows = x->volume() / std::max<size_t>(cols, 1);
  TTRT_ASSERT((!w || (w->volume() == cols && w->dtype == x->dtype)) && (!res || (res->volume() == x->volume() && res->dtype == x->dtype)) &&
                  out->dtype == x->dtype && out->volume() == x->volume(),
              "distributed_rms_norm operands must match the input's local width and data type");
  const uint32_t n = meshAxisSize(op->cluster_axis());
  TensorPtr local = makeDeviceTensor(dev, {static_cast<uint32_t>(rows)}, DataType::Float32);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_norm_row_stats(x->shards[i]->ptr, res ? res->shards[i]->ptr : nullptr, local->shards[i]->ptr, ttbDtype(x->dtype),
                                ttbDtype(DataType::Float32), rows, cols, 2, r.stream));
  });
  TensorPtr total = local;
  if (n > 1) {
    total = makeDeviceTensor(dev, {static_cast<uint32_t>(rows)}, DataType::Float32);
    allReduce(local, nullptr, total, 0);
  }
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_rms_norm_apply(x->shards[i]->ptr, res ? res->shards[i]->ptr : nullptr, w ? w->shards[i]->ptr : nullptr, nullptr,
                                static_cast<const float *>(total->shards[i]->ptr), out->shards[i]->ptr, ttbDtype(x->dtype), rows, cols,
                                cols * n, op->epsilon(), 0, r.stream));
  });
  put(op->out(), out);
}

// rms_norm_pre_all_gather (mode 0) and layer_norm_pre_all_gather (mode 1): per-row statistics in tile layout.
void Executor::runNormPreAllGather(const fbt::TensorRef *inRef, const fbt::TensorRef *resRef, const fbt::TensorRef *outRef, int mode) {
  TensorPtr x = getDevice(inRef);
  TensorPtr res = resRef ? getDevice(resRef) : nullptr;
  TensorPtr out = allocOut(outRef);
  TTRT_ASSERT(!x->shape.empty(), "norm statistics of a scalar");
  const size_t cols = x->shape.back(), rows = x->volume() / std::max<size_t>(cols, 1);
  const size_t width = mode == 0 ? 32 : 64;
  TTRT_ASSERT(!res || (res->volume() == x->volume() && res->dtype == x->dtype), "the residual must have the input's shape and data type");
  TTRT_ASSERT(out->volume() == rows * width && out->shape.back() == width, "the statistics tensor must be [..., ", width, "]");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_norm_row_stats(x->shards[i]->ptr, res ? res->shards[i]->ptr : nullptr, out->shards[i]->ptr, ttbDtype(x->dtype),
                                ttbDtype(out->dtype), rows, cols, mode, r.stream));
  });
  put(outRef, out);
}

void Executor::runLayerNormPostAllGather(const fbt::LayerNormPostAllGatherOp *op) {
  TensorPtr x = getDevice(op->input()), stats = getDevice(op->stats());
  TensorPtr w = op->weight() ? getDevice(op->weight()) : nullptr, b = op->bias() ? getDevice(op->bias()) : nullptr;
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(!x->shape.empty() && !stats->shape.empty(), "layer norm of a scalar");
  const size_t cols = x->shape.back(), rows = x->volume() / std::max<size_t>(cols, 1);
  TTRT_ASSERT(stats->shape.back() % 64 == 0 && stats->volume() == rows * stats->shape.back(),
              "the gathered statistics must be [..., 64 x devices] with the input's rows");
  const size_t blocks = stats->shape.back() / 64;
  TTRT_ASSERT((!w || (w->volume() == cols && w->dtype == x->dtype)) && (!b || (b->volume() == cols && b->dtype == x->dtype)) &&
                  out->dtype == x->dtype && out->volume() == x->volume(),
              "layer_norm_post_all_gather operands must match the input's local width and data type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_layer_norm_post_all_gather(x->shards[i]->ptr, stats->shards[i]->ptr, w ? w->shards[i]->ptr : nullptr,
                                            b ? b->shards[i]->ptr : nullptr, out->shards[i]->ptr, ttbDtype(x->dtype),
                                            ttbDtype(stats->dtype), rows, cols, blocks, op->epsilon(), r.stream));
  });
  put(op->out(), out);
}

// A second name for the same memory (annotate, region markers).
void Executor::runAlias(const fbt::TensorRef *operand, const fbt::TensorRef *result) {
  TensorPtr in = get(operand);
  auto alias = std::make_shared<TensorImpl>();
  alias->shape = in->shape;
  alias->stride = in->stride;
  alias->dtype = in->dtype;
  alias->storage = in->storage;
  alias->layout = in->layout;
  alias->shards = in->shards;
  alias->device = in->device;
  alias->preparedFrom = in->preparedFrom;
  put(result, alias);
}

// assign: a copy of the input, in the result's data type when one is given (operations/data_movement/assign.cpp).
void Executor::runAssign(const fbt::AssignOp *op) {
  TensorPtr in = getDevice(op->input());
  DataType dt = op->output_dtype().value_or(in->dtype);
  TensorPtr out = dt != in->dtype ? castOnDevice(in, dt) : stridedView(in, in->shape, denseStrides(in->shape), 0, in->dtype);
  TTRT_ASSERT(out->volume() == prod(refShape(op->output()), 0, refShape(op->output()).size()), "assign changes the element count");
  put(op->output(), out);
}

// pow(x, scalar) (operations/eltwise/binary/binary_composite_scalar.cpp; golden tools/golden/mapping.py:10447-10450).
void Executor::runPowScalar(const fbt::EltwiseBinaryCompositeScalarOp *op) {
  TTRT_ASSERT(op->type() == fbt::EltwiseBinaryCompositeScalarOpType::PowScalar, "unknown scalar composite op");
  TensorPtr in = getDevice(op->lhs());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(out->volume() == in->volume(), "pow_scalar changes the element count");
  TTRT_ASSERT(in->dtype == DataType::Float32 || in->dtype == DataType::BFloat16 || in->dtype == DataType::Float16,
              "pow_scalar takes floating-point tensors");
  const float e = numberValue(op->rhs_type(), op->rhs());
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_eltwise_unary(202, in->shards[i]->ptr, ttbDtype(in->dtype), out->shards[i]->ptr, ttbDtype(out->dtype), out->volume(), e,
                               r.stream));
  });
  put(op->out(), out);
}

// dump_tensor / load_tensor (operations/tensor_serialization/{dump,load}_tensor.cpp).  The reference writes tt-metal's
// tensor flatbuffer, a format of its own library; a file written here is read back here.  Layout: "TTB200T1", data type
// (u32), rank (u32), dimensions (u32 each), shard count (u32), then per shard its index (u32), byte count (u64), bytes.
static const char kTensorFileMagic[8] = {'T', 'T', 'B', '2', '0', '0', 'T', '1'};

void Executor::runDumpTensor(const fbt::DumpTensorOp *op) {
  refuseWhileRecording("dump_tensor");
  TensorPtr t = get(op->in());
  TensorPtr h = t->storage == Storage::Device ? toHostTensor(t, true) : t;
  TTRT_ASSERT(op->file_path() != nullptr, "dump_tensor without a file path");
  const std::string path = op->file_path()->str();
  std::ofstream f(path, std::ios::binary | std::ios::trunc);
  TTRT_ASSERT(f.is_open(), "dump_tensor cannot open ", path);
  auto u32 = [&](uint32_t v) { f.write(reinterpret_cast<const char *>(&v), 4); };
  f.write(kTensorFileMagic, 8);
  u32(static_cast<uint32_t>(h->dtype));
  u32(static_cast<uint32_t>(h->shape.size()));
  for (uint32_t d : h->shape) u32(d);
  u32(static_cast<uint32_t>(h->shards.size()));
  for (size_t i = 0; i < h->shards.size(); ++i) {
    const BufferPtr &b = h->shards[i];
    const uint64_t n = b && b->ptr ? h->bytes() : 0;
    u32(static_cast<uint32_t>(i));
    f.write(reinterpret_cast<const char *>(&n), 8);
    if (n) f.write(static_cast<const char *>(b->ptr), static_cast<std::streamsize>(n));
  }
  TTRT_ASSERT(f.good(), "dump_tensor failed writing ", path);
}

void Executor::runLoadTensor(const fbt::LoadTensorOp *op) {
  refuseWhileRecording("load_tensor");
  TTRT_ASSERT(op->file_path() != nullptr, "load_tensor without a file path");
  const std::string path = op->file_path()->str();
  std::ifstream f(path, std::ios::binary);
  TTRT_ASSERT(f.is_open(), "load_tensor cannot open ", path);
  char magic[8];
  f.read(magic, 8);
  TTRT_ASSERT(f.good() && std::memcmp(magic, kTensorFileMagic, 8) == 0, path, " is not a tensor file of this runtime");
  auto u32 = [&]() {
    uint32_t v = 0;
    f.read(reinterpret_cast<char *>(&v), 4);
    return v;
  };
  const DataType dt = static_cast<DataType>(u32());
  const uint32_t rank = u32();
  TTRT_ASSERT(f.good() && rank <= 8 && isSupportedDataType(dt), path, ": bad tensor header");
  std::vector<uint32_t> shape(rank);
  for (uint32_t &d : shape) d = u32();
  const uint32_t nshards = u32();
  TTRT_ASSERT(f.good() && nshards >= 1 && nshards <= 64, path, ": bad shard count");
  TensorPtr h = makeHostTensor(shape, dt, nshards);
  for (uint32_t k = 0; k < nshards; ++k) {
    const uint32_t idx = u32();
    uint64_t n = 0;
    f.read(reinterpret_cast<char *>(&n), 8);
    TTRT_ASSERT(f.good() && idx < nshards && (n == 0 || n == h->bytes()), path, ": bad shard record");
    if (n) f.read(static_cast<char *>(h->shards[idx]->ptr), static_cast<std::streamsize>(n));
    TTRT_ASSERT(f.good(), path, " is truncated");
  }
  TTRT_ASSERT(shape == refShape(op->out()) && dt == refDtype(op->out()), "the tensor in ", path, " does not have the op's result type");
  h->layout = refLayout(op->out());
  put(op->out(), op->device() && refOnDevice(op->out()) ? toDevice(h, dev, dt) : h);
}

// memory_snapshot (operations/debug/debug.cpp:34-54) writes the allocator's state per buffer type to a file.  There is
// one kind of device memory here: the figures are those of each local GPU's default memory pool and of the device.
void Executor::runMemorySnapshot(const fbt::MemorySnapshotOp *op) {
  TTRT_ASSERT(op->file_path() != nullptr, "memory_snapshot without a file path");
  const std::string path = op->file_path()->str();
  std::ofstream f(path, std::ios::out | std::ios::trunc);
  if (!f.is_open()) TTRT_FATAL("Failed to open file: ", path);
  eachRank([&](size_t, const RankCtx &r) {
    uint64_t reserved = 0, used = 0, high = 0;
    TTB_CALL(ttb_mempool_stats(&reserved, &used, &high, 0));
    int sms = 0, major = 0, minor = 0;
    size_t total = 0;
    TTB_CALL(ttb_device_info(r.cudaDevice, &sms, &total, &major, &minor));
    f << "Device " << r.meshRank << " DRAM memory state: totalBytes=" << total << " poolReservedBytes=" << reserved
      << " allocatedBytes=" << used << " peakAllocatedBytes=" << high << "\n";
  });
}

void Executor::runAllReduceAsync(const fbt::AllReduceAsyncOp *op) {
  TensorPtr in = getDevice(op->in());
  if (meshAxisSize(op->cluster_axis()) == 1) {
    put(op->out(), in);
    return;
  }
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(out->volume() == in->volume() && out->dtype == in->dtype, "all_reduce_async changes shape or type");
  allReduce(in, nullptr, out, static_cast<int>(op->reduce_type()));
  put(op->out(), out);
}

// point_to_point (operations/ccl/point_to_point.cpp): the result is the optional output tensor (or a copy of the input)
// on every coordinate, except that the receiver's shard is the sender's shard of the input.
void Executor::runPointToPoint(const fbt::PointToPointOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr base = op->optional_output_tensor() ? getDevice(op->optional_output_tensor()) : in;
  TTRT_ASSERT(base->dtype == in->dtype && base->volume() == in->volume(), "point_to_point output tensor differs from the input's type");
  auto linear = [&](const fb::Vector<uint32_t> *c, const char *what) {
    TTRT_ASSERT(c && c->size() == 2, "point_to_point ", what, " must be a 2-D mesh coordinate");
    TTRT_ASSERT(c->Get(0) < dev->meshShape[0] && c->Get(1) < dev->meshShape[1], "point_to_point ", what, " lies outside the mesh");
    return c->Get(0) * dev->meshShape[1] + c->Get(1);
  };
  const uint32_t sender = linear(op->sender_coord(), "sender_coord"), receiver = linear(op->receiver_coord(), "receiver_coord");
  TensorPtr out = stridedView(base, in->shape, denseStrides(in->shape), 0, in->dtype);
  if (sender != receiver) {
    refuseWhileRecording("a collective");
    TTB_CALL(ttb_group_start());
    eachRank([&](size_t i, const RankCtx &r) {
      if (r.meshRank == sender) {
        TTB_CALL(ttb_send(r.comm, in->shards[i]->ptr, in->volume(), ttbDtype(in->dtype), static_cast<int>(receiver), r.stream));
      }
      if (r.meshRank == receiver) {
        TTB_CALL(ttb_recv(r.comm, out->shards[i]->ptr, in->volume(), ttbDtype(in->dtype), static_cast<int>(sender), r.stream));
      }
    });
    TTB_CALL(ttb_group_end());
  } else {
    eachRank([&](size_t i, const RankCtx &r) {
      if (r.meshRank == receiver && base != in) {
        TTB_CALL(ttb_memcpy_d2d(out->shards[i]->ptr, in->shards[i]->ptr, in->bytes(), r.stream));
      }
    });
  }
  put(op->out(), out);
}

// nlp_create_qkv_heads_decode (operations/transformer/nlp_create_qkv_heads_decode.cpp): the fused projection of one
// decode step, [1, 1, batch, (Hq + 2 Hkv) * D], split into q [1, batch, Hq, D], k and v [1, batch, Hkv, D].  With
// `slice_size`, only the batch rows [batch_offset, batch_offset + slice_size) are taken.
void Executor::runNlpCreateQkvHeadsDecode(const fbt::NLPCreateQKVHeadsDecodeOp *op) {
  TensorPtr in = getDevice(op->input());
  TTRT_ASSERT(in->shape.size() == 4 && in->shape[0] == 1 && in->shape[1] == 1, "nlp_create_qkv_heads_decode expects [1, 1, batch, hidden]");
  const uint32_t B = in->shape[2], hidden = in->shape[3];
  const uint32_t Hq = op->num_heads(), Hkv = op->num_kv_heads().value_or(Hq);
  TTRT_ASSERT(Hq > 0 && Hkv > 0 && hidden % (Hq + 2 * Hkv) == 0, "hidden size ", hidden, " does not split into ", Hq, " + 2 x ", Hkv, " heads");
  const uint32_t D = hidden / (Hq + 2 * Hkv);
  uint32_t first = 0, count = B;
  if (op->slice_size().has_value()) {
    TTRT_ASSERT(op->batch_offset() != nullptr, "slice_size needs a batch_offset tensor");
    refuseWhileRecording("reading batch_offset");
    TensorPtr off = get(op->batch_offset());
    TTRT_ASSERT(off->volume() >= 1 && dataTypeSize(off->dtype) == 4, "batch_offset must hold one 32-bit integer");
    if (off->storage == Storage::Device) off = toHostTensor(off, true);
    first = *static_cast<const uint32_t *>(off->shards[0]->ptr);
    count = *op->slice_size();
    TTRT_ASSERT(static_cast<uint64_t>(first) + count <= B, "batch slice [", first, ", ", first + count, ") exceeds the batch of ", B);
  }
  auto heads = [&](uint32_t colOff, uint32_t H) {
    return stridedView(in, {1, count, H, D}, {0, static_cast<int64_t>(hidden), static_cast<int64_t>(D), 1},
                       static_cast<int64_t>(first) * hidden + colOff, in->dtype);
  };
  TensorPtr q = heads(0, Hq), k = heads(Hq * D, Hkv), v = heads((Hq + Hkv) * D, Hkv);
  TTRT_ASSERT(q->shape == refShape(op->q_out()) && k->shape == refShape(op->k_out()) && v->shape == refShape(op->v_out()),
              "nlp_create_qkv_heads_decode result shapes differ from the op's result types");
  put(op->q_out(), q);
  put(op->k_out(), k);
  put(op->v_out(), v);
}

// nlp_concat_heads_decode (operations/transformer/nlp_concat_heads_decode.cpp): [1, batch, padded heads, D] ->
// [1, 1, batch, num_heads * D], dropping the heads beyond `num_heads`.
void Executor::runNlpConcatHeadsDecode(const fbt::NLPConcatHeadsDecodeOp *op) {
  TensorPtr in = getDevice(op->in());
  TTRT_ASSERT(in->shape.size() == 4 && in->shape[0] == 1, "nlp_concat_heads_decode expects [1, batch, heads, head_dim]");
  const uint32_t B = in->shape[1], Hp = in->shape[2], D = in->shape[3], H = op->num_heads();
  TTRT_ASSERT(H >= 1 && H <= Hp, "num_heads ", H, " exceeds the input's ", Hp, " heads");
  TensorPtr t = stridedView(in, {B, H, D}, {static_cast<int64_t>(Hp) * D, static_cast<int64_t>(D), 1}, 0, in->dtype);
  t->shape = {1, 1, B, H * D};
  t->stride = denseStrides(t->shape);
  TTRT_ASSERT(t->shape == refShape(op->out()), "nlp_concat_heads_decode result shape differs from the op's result type");
  put(op->out(), t);
}

// rotary_embedding_llama (operations/transformer/rotary_embedding_llama.cpp).  Prefill: x [1, heads, seq, D] with caches
// [1, 1, seq, D].  Decode: x [1, batch, heads, D] with caches [1, batch, 1 or heads, D].
void Executor::runRotaryEmbeddingLlama(const fbt::RotaryEmbeddingLlamaOp *op) {
  TensorPtr x = getDevice(op->input()), c = getDevice(op->cos_cache()), s = getDevice(op->sin_cache()), t = getDevice(op->trans_mat());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(x->shape.size() >= 2 && c->shape == s->shape, "rotary_embedding_llama: cos and sin caches must have the same shape");
  const size_t rank = x->shape.size(), D = x->shape[rank - 1], inner = x->shape[rank - 2];
  const size_t rows = x->volume() / std::max<size_t>(D, 1);
  TTRT_ASSERT(t->volume() >= 1024 && t->shape.back() == 32, "the transformation matrix must be [1, 1, 32, 32]");
  TTRT_ASSERT(c->shape.back() == D && c->volume() % D == 0, "cache rows must have the head dimension ", D);
  TTRT_ASSERT(x->dtype == c->dtype && x->dtype == s->dtype && x->dtype == t->dtype && x->dtype == out->dtype && out->volume() == x->volume(),
              "rotary_embedding_llama tensors must share one data type");
  const size_t cacheRows = c->volume() / D;
  size_t mod = cacheRows, div = 1;
  if (op->is_decode_mode()) {
    // rows are (batch, head): one cache row per batch entry, or one per (batch, head)
    TTRT_ASSERT(cacheRows * inner == rows || cacheRows == rows, "decode caches must be [1, batch, 1, D] for x [1, batch, heads, D]");
    div = cacheRows == rows ? 1 : inner;
  } else {
    TTRT_ASSERT(cacheRows >= inner, "prefill caches hold ", cacheRows, " positions, the input has ", inner);
    mod = inner; // rows are (..., seq): position = row % seq
  }
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_rotary_embedding_llama(x->shards[i]->ptr, c->shards[i]->ptr, s->shards[i]->ptr, t->shards[i]->ptr, out->shards[i]->ptr,
                                        ttbDtype(x->dtype), rows, D, mod, div, r.stream));
  });
  put(op->out(), out);
}

void Executor::runMaxPool2dWithIndices(const fbt::MaxPool2dWithIndicesOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->result()), idx = allocOut(op->result_indices());
  const int n = static_cast<int>(op->batch_size()), h = static_cast<int>(op->input_height()), w = static_cast<int>(op->input_width()),
            c = static_cast<int>(op->channels());
  TTRT_ASSERT(in->volume() == size_t(n) * h * w * c, "max_pool2d_with_indices input has ", in->volume(), " elements, the op says ", n, "x",
              h, "x", w, "x", c);
  auto two = [](const fb::Vector<int32_t> *v, const char *what, int &a, int &b, int dflt) {
    if (!v || v->size() == 0) {
      a = b = dflt;
      return;
    }
    TTRT_ASSERT(v->size() == 2 || v->size() == 4, what, " needs two entries");
    a = v->Get(0);
    b = v->Get(1);
    if (v->size() == 4) TTRT_ASSERT(v->Get(2) == a && v->Get(3) == b, what, ": asymmetric padding is not supported with indices");
  };
  int kh, kw, sh, sw, ph, pw, dh, dw;
  two(op->kernel_size(), "kernel_size", kh, kw, 1);
  two(op->stride(), "stride", sh, sw, 1);
  two(op->padding(), "padding", ph, pw, 0);
  two(op->dilation(), "dilation", dh, dw, 1);
  int ho = 0, wo = 0;
  TTB_CALL(ttb_pool2d_out_shape(1, h, w, kh, kw, sh, sw, ph, pw, ph, pw, dh, dw, op->ceil_mode(), 0, &ho, &wo));
  TTRT_ASSERT(out->volume() == size_t(n) * ho * wo * c && idx->volume() == out->volume(), "max_pool2d_with_indices results have ",
              out->volume(), " elements, expected ", n, "x", ho, "x", wo, "x", c);
  TTRT_ASSERT(out->dtype == in->dtype, "max_pool2d_with_indices changes the data type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_max_pool2d_with_indices(in->shards[i]->ptr, out->shards[i]->ptr, idx->shards[i]->ptr, ttbDtype(in->dtype),
                                         ttbDtype(idx->dtype), n, h, w, c, ho, wo, kh, kw, sh, sw, ph, pw, dh, dw, r.stream));
  });
  put(op->result(), out);
  put(op->result_indices(), idx);
}

// dropout: with use_per_device_seed every mesh coordinate draws its own stream (operations/eltwise/unary/dropout.cpp).
void Executor::runDropout(const fbt::DropoutOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(out->dtype == in->dtype && out->volume() == in->volume(), "dropout changes shape or type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_dropout(in->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(in->dtype), in->volume(), op->prob(), op->scale(), op->seed(),
                         op->use_per_device_seed() ? r.meshRank : 0u, r.stream));
  });
  put(op->out(), out);
}

// rand: uniform in [low, high), the same tensor on every mesh coordinate (golden mapping.py:4340-4362).
void Executor::runRand(const fbt::RandOp *op) {
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(op->size() != nullptr, "rand without a size");
  size_t n = 1;
  for (int64_t d : *op->size()) n *= static_cast<size_t>(d);
  TTRT_ASSERT(n == out->volume(), "rand size differs from the op's result type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_rand_uniform(out->shards[i]->ptr, ttbDtype(out->dtype), n, op->low(), op->high(), op->seed(), 0u, r.stream));
  });
  put(op->out(), out);
}

// Training batch norm over dim 1 of [N, C, ...]; running_mean / running_var are updated in place.
void Executor::runBatchNormTraining(const fbt::BatchNormTrainingOp *op) {
  TensorPtr x = getDevice(op->input()), mean = getDevice(op->running_mean()), var = getDevice(op->running_var());
  TensorPtr w = op->weight() ? getDevice(op->weight()) : nullptr, b = op->bias() ? getDevice(op->bias()) : nullptr;
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(x->shape.size() >= 2, "batch_norm expects [N, C, ...]");
  const size_t outer = x->shape[0], channels = x->shape[1], inner = prod(x->shape, 2, x->shape.size());
  TTRT_ASSERT(mean->volume() == channels && var->volume() == channels && (!w || w->volume() == channels) && (!b || b->volume() == channels),
              "batch_norm statistics and parameters must have one entry per channel (", channels, ")");
  TTRT_ASSERT(mean->dtype == x->dtype && var->dtype == x->dtype && (!w || w->dtype == x->dtype) && (!b || b->dtype == x->dtype) &&
                  out->dtype == x->dtype && out->volume() == x->volume(),
              "batch_norm tensors must share one data type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_batch_norm_training(x->shards[i]->ptr, mean->shards[i]->ptr, var->shards[i]->ptr, w ? w->shards[i]->ptr : nullptr,
                                     b ? b->shards[i]->ptr : nullptr, out->shards[i]->ptr, ttbDtype(x->dtype), outer, channels, inner,
                                     op->epsilon(), op->momentum(), r.stream));
  });
  mean->version = TensorImpl::nextTensorVersion();
  var->version = TensorImpl::nextTensorVersion();
  put(op->out(), out);
}

// group_norm on channels-last [N, 1, H*W, C] (or [N, H, W, C]): operations/normalization/group_norm.cpp.
void Executor::runGroupNorm(const fbt::GroupNormOp *op) {
  TTRT_ASSERT(!op->input_mask(), "group_norm with an input mask (a Tenstorrent core-grid artefact) is not supported");
  TensorPtr x = getDevice(op->input());
  TensorPtr w = op->weight() ? getDevice(op->weight()) : nullptr, b = op->bias() ? getDevice(op->bias()) : nullptr;
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(x->shape.size() == 4, "group_norm expects [N, 1, H*W, C]");
  const size_t images = x->shape[0], channels = x->shape[3], pixels = static_cast<size_t>(x->shape[1]) * x->shape[2];
  const size_t groups = static_cast<size_t>(op->num_groups());
  TTRT_ASSERT(groups >= 1 && channels % groups == 0, "group_norm: ", channels, " channels do not divide into ", groups, " groups");
  TTRT_ASSERT((!w || (w->volume() == channels && w->dtype == x->dtype)) && (!b || (b->volume() == channels && b->dtype == x->dtype)) &&
                  out->dtype == x->dtype && out->volume() == x->volume(),
              "group_norm parameters must have one entry per channel and the input's data type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_group_norm(x->shards[i]->ptr, w ? w->shards[i]->ptr : nullptr, b ? b->shards[i]->ptr : nullptr, out->shards[i]->ptr,
                            ttbDtype(x->dtype), images, pixels, channels, groups, op->epsilon(), r.stream));
  });
  put(op->out(), out);
}

// conv_transpose2d on NHWC activations (flattened to [1, 1, N*H*W, C] or not), weights [C_in, C_out / groups, kH, kW].
void Executor::runConvTranspose2d(const fbt::ConvTranspose2dOp *op) {
  TensorPtr x = getDevice(op->input()), w = getDevice(op->weight());
  TensorPtr bias = op->bias() ? getDevice(op->bias()) : nullptr;
  if (w->preparedFrom) w = w->preparedFrom; // prepare_conv_transpose2d_weights handed the original on
  if (bias && bias->preparedFrom) bias = bias->preparedFrom;
  TensorPtr out = allocOut(op->out());
  auto two = [](const fb::Vector<int32_t> *v, const char *what, int &a, int &b) {
    TTRT_ASSERT(v && (v->size() == 2 || v->size() == 4), "conv_transpose2d ", what, " must have 2 entries");
    a = v->Get(0);
    b = v->Get(1);
  };
  int kh, kw, sh, sw, ph, pw, oph, opw, dh, dw;
  two(op->kernel_size(), "kernel_size", kh, kw);
  two(op->stride(), "stride", sh, sw);
  two(op->padding(), "padding", ph, pw);
  two(op->output_padding(), "output_padding", oph, opw);
  two(op->dilation(), "dilation", dh, dw);
  const int64_t N = op->batch_size(), H = op->input_height(), W = op->input_width(), C = op->in_channels(), O = op->out_channels();
  TTRT_ASSERT(static_cast<int64_t>(x->volume()) == N * H * W * C, "conv_transpose2d input has ", x->volume(), " elements, expected ",
              N * H * W * C);
  TTRT_ASSERT(x->dtype == w->dtype && x->dtype == out->dtype && (!bias || bias->dtype == x->dtype),
              "conv_transpose2d tensors must share one data type");
  const int64_t ho = (H - 1) * sh - 2 * ph + dh * (kh - 1) + oph + 1, wo = (W - 1) * sw - 2 * pw + dw * (kw - 1) + opw + 1;
  TTRT_ASSERT(static_cast<int64_t>(out->volume()) == N * ho * wo * O, "conv_transpose2d result has ", out->volume(),
              " elements, expected ", N * ho * wo * O);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_conv_transpose2d(x->shards[i]->ptr, w->shards[i]->ptr, bias ? bias->shards[i]->ptr : nullptr, out->shards[i]->ptr,
                                  ttbDtype(x->dtype), N, H, W, C, O, kh, kw, sh, sw, ph, pw, oph, opw, dh, dw,
                                  static_cast<int>(op->groups()), r.stream));
  });
  put(op->out(), out);
}

// conv1d over [N, L, C] activations (flattened or not) with weights [O, C / groups, K]: a conv2d with one row.
void Executor::runConv1d(const fbt::Conv1dOp *op) {
  TensorPtr x = getDevice(op->input()), w = getDevice(op->weight());
  TensorPtr bias = op->bias() ? getDevice(op->bias()) : nullptr;
  TensorPtr out = allocOut(op->out());
  const int64_t N = op->batch_size(), L = op->input_length(), C = op->in_channels(), O = op->out_channels();
  const int K = static_cast<int>(op->kernel_size()), stride = static_cast<int>(op->stride()), dil = static_cast<int>(op->dilation());
  TTRT_ASSERT(op->padding() && (op->padding()->size() == 1 || op->padding()->size() == 2), "conv1d padding must have 1 or 2 entries");
  const int pl = op->padding()->Get(0), pr = op->padding()->size() == 2 ? op->padding()->Get(1) : pl;
  int pad[4] = {0, pl, 0, pr}; // top, left, bottom, right
  TTRT_ASSERT(static_cast<int64_t>(x->volume()) == N * L * C, "conv1d input has ", x->volume(), " elements, expected ", N * L * C);
  TTRT_ASSERT(x->dtype == w->dtype && x->dtype == out->dtype, "conv1d tensors must share one data type");
  const int groups = static_cast<int>(op->groups());
  size_t wsBytes = ttb_conv2d_workspace_bytes(ttbDtype(x->dtype), N, 1, L, C, O, 1, K, 1, stride, pad, 1, dil, groups);
  TensorPtr ws = wsBytes ? makeDeviceTensor(dev, {static_cast<uint32_t>((wsBytes + 3) / 4)}, DataType::UInt32) : nullptr;
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_conv2d_fused(x->shards[i]->ptr, w->shards[i]->ptr, bias ? bias->shards[i]->ptr : nullptr, out->shards[i]->ptr,
                              ttbDtype(x->dtype), bias ? ttbDtype(bias->dtype) : 0, N, 1, L, C, O, 1, K, 1, stride, pad, 1, dil, groups,
                              TTB_ACT_NONE, nullptr, TTB_EXTRA_NONE, ws ? ws->shards[i]->ptr : nullptr, r.stream));
  });
  put(op->out(), out);
}

// bitcast_convert: the same bytes under another element type of the same width (operations/layout/bitcast_convert.cpp).
void Executor::runBitcastConvert(const fbt::BitcastConvertOp *op) {
  TensorPtr in = getDevice(op->in());
  TTRT_ASSERT(dataTypeSize(op->dtype()) == dataTypeSize(in->dtype), "bitcast_convert between types of different widths");
  auto view = std::make_shared<TensorImpl>();
  view->shape = refShape(op->out());
  view->stride = denseStrides(view->shape);
  view->dtype = op->dtype();
  view->storage = in->storage;
  view->layout = refLayout(op->out());
  view->shards = in->shards;
  view->device = in->device;
  TTRT_ASSERT(view->volume() == in->volume(), "bitcast_convert changes the element count");
  put(op->out(), view);
}

// [B, H, S, D] -> [B, 1, S, H*D] (operations/transformer/nlp_concat_heads.cpp): concatenate_heads with a unit dimension.
void Executor::runNlpConcatHeads(const fbt::NLPConcatHeadsOp *op) {
  TensorPtr in = getDevice(op->in());
  TTRT_ASSERT(in->shape.size() == 4, "nlp_concat_heads expects [batch, heads, seq, head_dim]");
  uint32_t B = in->shape[0], H = in->shape[1], S = in->shape[2], D = in->shape[3];
  std::vector<int64_t> dense = denseStrides(in->shape);
  TensorPtr t = stridedView(in, {B, S, H, D}, {dense[0], dense[2], dense[1], dense[3]}, 0, in->dtype);
  t->shape = {B, 1, S, H * D};
  t->stride = denseStrides(t->shape);
  TTRT_ASSERT(t->shape == refShape(op->out()), "nlp_concat_heads result shape differs from the op's result type");
  put(op->out(), t);
}

// Inference batch norm over the channel dimension (dim 1, NCHW, as ::ttnn::batch_norm takes it).
void Executor::runBatchNormInference(const fbt::BatchNormInferenceOp *op) {
  TensorPtr x = getDevice(op->input()), mean = getDevice(op->running_mean()), var = getDevice(op->running_var());
  TensorPtr w = op->weight() ? getDevice(op->weight()) : nullptr, b = op->bias() ? getDevice(op->bias()) : nullptr;
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(x->shape.size() >= 2, "batch_norm expects [N, C, ...]");
  const size_t outer = x->shape[0], channels = x->shape[1], inner = prod(x->shape, 2, x->shape.size());
  TTRT_ASSERT(mean->volume() == channels && var->volume() == channels && (!w || w->volume() == channels) &&
                  (!b || b->volume() == channels),
              "batch_norm statistics and parameters must have one entry per channel (", channels, ")");
  TTRT_ASSERT(mean->dtype == x->dtype && var->dtype == x->dtype && (!w || w->dtype == x->dtype) && (!b || b->dtype == x->dtype) &&
                  out->dtype == x->dtype && out->volume() == x->volume(),
              "batch_norm tensors must share one data type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_batch_norm_inference(x->shards[i]->ptr, mean->shards[i]->ptr, var->shards[i]->ptr, w ? w->shards[i]->ptr : nullptr,
                                      b ? b->shards[i]->ptr : nullptr, out->shards[i]->ptr, ttbDtype(x->dtype), outer, channels,
                                      inner, op->epsilon(), r.stream));
  });
  put(op->out(), out);
}

// NHWC upsampling by integer factors, "nearest" or "bilinear" (operations/pool/upsample.cpp).
void Executor::runUpsample(const fbt::UpsampleOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(in->shape.size() == 4, "upsample expects [N, H, W, C]");
  int sy = 1, sx = 1;
  if (const auto *u = op->scale_factor_as_UniformScale2D()) {
    sy = sx = u->scale();
  } else if (const auto *nu = op->scale_factor_as_NonUniformScale2D()) {
    TTRT_ASSERT(nu->scale() && nu->scale()->size() == 2, "upsample scale must have 2 entries");
    sy = nu->scale()->Get(0);
    sx = nu->scale()->Get(1);
  } else {
    TTRT_FATAL("upsample without a scale factor");
  }
  const std::string mode = op->mode() ? op->mode()->str() : "nearest";
  TTRT_ASSERT(mode == "nearest" || mode == "bilinear", "upsample mode ", mode, " is not supported");
  TTRT_ASSERT(sy >= 1 && sx >= 1 && out->dtype == in->dtype && out->shape.size() == 4 && out->shape[0] == in->shape[0] &&
                  out->shape[1] == in->shape[1] * static_cast<uint32_t>(sy) && out->shape[2] == in->shape[2] * static_cast<uint32_t>(sx) &&
                  out->shape[3] == in->shape[3],
              "upsample result shape differs from input x scale");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_upsample2d(in->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(in->dtype), in->shape[0], in->shape[1], in->shape[2],
                            in->shape[3], sy, sx, mode == "bilinear" ? 1 : 0, r.stream));
  });
  put(op->out(), out);
}

// prepare_conv2d_weights / prepare_conv2d_bias: TTNN re-tiles and shards the tensor for its convolution kernels and
// the flatbuffer declares that layout's shape; nothing of it applies here.  The result keeps the declared shape as
// metadata and carries the tensor it was made from, which is what conv2d then reads.
void Executor::runPrepareConv2d(const fbt::TensorRef *inRef, const fbt::TensorRef *outRef) {
  TensorPtr in = getDevice(inRef);
  auto t = std::make_shared<TensorImpl>();
  t->shape = refShape(outRef);
  t->stride = denseStrides(t->shape);
  t->dtype = in->dtype;
  t->storage = in->storage;
  t->layout = refLayout(outRef);
  t->shards = in->shards;
  t->device = in->device;
  t->preparedFrom = in->preparedFrom ? in->preparedFrom : in;
  put(outRef, t);
}

// out[..., :] = weight[input[...], :]; a weight of shape [1, 1, V, D] is a [V, D] table.
void Executor::runEmbedding(const fbt::EmbeddingOp *op) {
  TensorPtr idx = getDevice(op->input());
  TensorPtr w = getDevice(op->weight());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(w->shape.size() >= 2, "embedding table needs two dimensions");
  size_t dim = w->shape.back(), vocab = w->shape[w->shape.size() - 2];
  TTRT_ASSERT(w->volume() == vocab * dim, "embedding table has leading dimensions other than 1");
  TTRT_ASSERT(out->dtype == w->dtype, "embedding result must have the table's data type");
  size_t rows = idx->volume();
  dev->ranEmbedding = true;
  TTRT_ASSERT(out->volume() == rows * dim, "embedding result has ", out->volume(), " elements, expected ", rows * dim);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_embedding(idx->shards[i]->ptr, w->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(idx->dtype), ttbDtype(w->dtype),
                           rows, vocab, dim, r.stream));
  });
  put(op->out(), out);
}

// Pool2dOp: NHWC activation, flattened to [1, 1, N*H*W, C] in real flatbuffers; N, H, W, C come as fields.
void Executor::runPool2d(const fbt::Pool2dOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  const int n = static_cast<int>(op->batch_size()), h = static_cast<int>(op->input_height()),
            w = static_cast<int>(op->input_width()), c = static_cast<int>(op->channels());
  TTRT_ASSERT(in->volume() == size_t(n) * h * w * c, "pool2d input has ", in->volume(), " elements, the op says ", n, "x", h,
              "x", w, "x", c);
  auto two = [](const fb::Vector<int32_t> *v, const char *what, int &a, int &b, int dflt) {
    if (!v || v->size() == 0) {
      a = b = dflt;
      return;
    }
    TTRT_ASSERT(v->size() == 2, what, " needs two entries");
    a = v->Get(0);
    b = v->Get(1);
  };
  int kh, kw, sh, sw, dh, dw;
  two(op->kernel_size(), "kernel_size", kh, kw, 1);
  two(op->stride(), "stride", sh, sw, 1);
  two(op->dilation(), "dilation", dh, dw, 1);
  int pt = 0, pl = 0, pb = 0, pr = 0, four = 0;
  if (op->padding() && op->padding()->size() == 2) {
    pt = pb = op->padding()->Get(0);
    pl = pr = op->padding()->Get(1);
  } else if (op->padding() && op->padding()->size() == 4) {
    pt = op->padding()->Get(0); // top, left, bottom, right (runtime/lib/ttnn/operations/pool/pool2d.cpp:49-55)
    pl = op->padding()->Get(1);
    pb = op->padding()->Get(2);
    pr = op->padding()->Get(3);
    four = 1;
  } else {
    TTRT_ASSERT(!op->padding() || op->padding()->size() == 0, "padding needs two or four entries");
  }
  const bool isMax = op->type() == fbt::Pool2dOpType::MaxPool2d;
  int includePad = 1;
  if (!isMax) {
    const auto *extra = op->extra_params_as_AvgPool2dExtraParams();
    TTRT_ASSERT(extra != nullptr, "avg_pool2d without its parameters");
    includePad = extra->count_include_pad() ? 1 : 0;
  }
  int ho = 0, wo = 0;
  TTB_CALL(ttb_pool2d_out_shape(isMax, h, w, kh, kw, sh, sw, pt, pl, pb, pr, isMax ? dh : 1, isMax ? dw : 1, op->ceil_mode(), four,
                                &ho, &wo));
  TTRT_ASSERT(out->volume() == size_t(n) * ho * wo * c, "pool2d result has ", out->volume(), " elements, expected ", n, "x", ho,
              "x", wo, "x", c);
  TTRT_ASSERT(out->dtype == in->dtype, "pool2d changes the data type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_pool2d(in->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(in->dtype), isMax, n, h, w, c, kh, kw, sh, sw, pt, pl,
                        pb, pr, dh, dw, op->ceil_mode(), includePad, four, r.stream));
  });
  put(op->out(), out);
}

// [N, H, W, C] -> [N, 1, 1, C]: the mean over H*W, which is the column form of the reduction kernel.
void Executor::runGlobalAvgPool2d(const fbt::GlobalAvgPool2dOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(in->shape.size() == 4, "global_avg_pool2d expects an NHWC tensor");
  TTRT_ASSERT(out->dtype == in->dtype, "global_avg_pool2d with a type change is not supported");
  size_t n = in->shape[0], hw = size_t(in->shape[1]) * in->shape[2], c = in->shape[3];
  TTRT_ASSERT(out->volume() == n * c, "global_avg_pool2d result has ", out->volume(), " elements, expected ", n * c);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_reduce(1 /* mean */, in->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(in->dtype), n, hw, c, r.stream));
  });
  put(op->out(), out);
}

void Executor::runPad(const fbt::PadOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr out = allocOut(op->out());
  size_t rank = in->shape.size();
  TTRT_ASSERT(rank >= 1 && rank <= 8, "pad supports ranks 1 to 8");
  TTRT_ASSERT(op->padding() && op->padding()->size() == 2 * rank, "pad needs a (low, high) pair per dimension");
  int64_t shape[8], lo[8], hi[8];
  size_t vol = 1;
  for (size_t d = 0; d < rank; ++d) {
    shape[d] = in->shape[d];
    lo[d] = op->padding()->Get(static_cast<uint32_t>(2 * d));
    hi[d] = op->padding()->Get(static_cast<uint32_t>(2 * d + 1));
    vol *= static_cast<size_t>(shape[d] + lo[d] + hi[d]);
  }
  TTRT_ASSERT(out->volume() == vol && out->dtype == in->dtype, "pad result does not match input plus padding");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_pad(in->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(in->dtype), static_cast<int>(rank), shape, lo, hi,
                     static_cast<double>(op->value()), r.stream));
  });
  put(op->out(), out);
}

// ---- KV cache --------------------------------------------------------------------------------------------------
// FillCacheOp / UpdateCacheOp write into the cache tensor in place (they have no result); the
// tensor's version is renewed, so traces and const-eval entries keyed by it notice.
void Executor::runFillCache(const fbt::FillCacheOp *op) {
  TensorPtr cache = getDevice(op->cache());
  TensorPtr in = getDevice(op->input());
  TTRT_ASSERT(cache->shape.size() == 4 && in->shape.size() == 4, "fill_cache expects [users, heads, seq, head_dim] tensors");
  TTRT_ASSERT(cache->dtype == in->dtype, "fill_cache input must have the cache's data type");
  TTRT_ASSERT(in->shape[1] == cache->shape[1] && in->shape[3] == cache->shape[3], "fill_cache input does not match the cache's heads / head_dim");
  TTRT_ASSERT(in->shape[2] <= cache->shape[2], "fill_cache input is longer than the cache");
  TTRT_ASSERT(op->batch_offset() + in->shape[0] <= cache->shape[0], "fill_cache input users do not fit the cache");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_fill_cache(cache->shards[i]->ptr, in->shards[i]->ptr, ttbDtype(cache->dtype), in->shape[0], in->shape[1],
                            in->shape[2], cache->shape[2], cache->shape[3], op->batch_offset(), cache->shape[0], r.stream));
  });
  TensorPtr root = cache->base ? cache->base : cache;
  root->version.store(TensorImpl::nextTensorVersion());
}

void Executor::runUpdateCache(const fbt::UpdateCacheOp *op) {
  TensorPtr cache = getDevice(op->cache());
  TensorPtr in = getDevice(op->input());
  TensorPtr idx = getDevice(op->update_index()); // read by the kernel: no host round trip
  TTRT_ASSERT(cache->shape.size() == 4 && in->shape.size() == 4, "update_cache expects 4-D tensors");
  TTRT_ASSERT(cache->dtype == in->dtype, "update_cache input must have the cache's data type");
  TTRT_ASSERT(in->shape[0] == 1 && in->shape[1] == cache->shape[1] && in->shape[3] == cache->shape[3],
              "update_cache input must be [1, heads, users, head_dim]");
  TTRT_ASSERT(op->batch_offset() + in->shape[2] <= cache->shape[0], "update_cache input users do not fit the cache");
  dev->ranUpdateCache = true;
  TTRT_ASSERT(idx->volume() >= 1 && (idx->dtype == DataType::Int32 || idx->dtype == DataType::UInt32),
              "update_cache index must be an Int32 / UInt32 tensor");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_update_cache(cache->shards[i]->ptr, in->shards[i]->ptr, idx->shards[i]->ptr, ttbDtype(cache->dtype),
                              ttbDtype(idx->dtype), in->shape[2], in->shape[1], cache->shape[2], cache->shape[3],
                              op->batch_offset(), cache->shape[0], r.stream));
  });
  TensorPtr root = cache->base ? cache->base : cache;
  root->version.store(TensorImpl::nextTensorVersion());
}

// q [1, B, H, D] against k, v [B, Hkv, S, D] (the decode layout, tools/golden/mapping.py:2431-2437).
void Executor::runSdpaDecode(const fbt::ScaledDotProductAttentionDecodeOp *op) {
  TTRT_ASSERT(!op->attention_sink(), "attention sinks are not supported");
  TTRT_ASSERT(!op->sliding_window_size().has_value(), "sliding-window decode attention is not supported");
  TensorPtr q = getDevice(op->query()), k = getDevice(op->key()), v = getDevice(op->value());
  TensorPtr mask = op->attention_mask() ? getDevice(op->attention_mask()) : nullptr;
  TensorPtr pos = op->cur_pos_tensor() ? getDevice(op->cur_pos_tensor()) : nullptr;
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(q->shape.size() == 4 && k->shape.size() == 4 && v->shape == k->shape, "sdpa_decode expects q [1,B,H,D], k / v [B,Hkv,S,D]");
  TTRT_ASSERT(q->shape[0] == 1 && q->shape[1] == k->shape[0] && q->shape[3] == k->shape[3], "sdpa_decode operands disagree on batch or head_dim");
  TTRT_ASSERT(q->dtype == k->dtype && q->dtype == v->dtype && out->dtype == q->dtype, "sdpa_decode operands must share one data type");
  const int B = static_cast<int>(q->shape[1]), H = static_cast<int>(q->shape[2]), D = static_cast<int>(q->shape[3]);
  const int Hkv = static_cast<int>(k->shape[1]), S = static_cast<int>(k->shape[2]);
  TTRT_ASSERT(out->volume() == q->volume(), "sdpa_decode result must have the query's shape");
  int maskB = 0, maskH = 0;
  if (mask) {
    TTRT_ASSERT(mask->shape.size() == 4 && mask->shape[1] == 1 && static_cast<int>(mask->shape[3]) == S && mask->dtype == q->dtype,
                "sdpa_decode mask must be [B or 1, 1, H or 1, S] in the operands' data type");
    maskB = static_cast<int>(mask->shape[0]);
    maskH = static_cast<int>(mask->shape[2]);
  }
  if (pos) {
    TTRT_ASSERT(static_cast<int>(pos->volume()) == B && (pos->dtype == DataType::Int32 || pos->dtype == DataType::UInt32),
                "cur_pos must hold one 32-bit integer per user");
  }
  // The golden applies no scaling when the op carries none (tools/golden/mapping.py:2471-2473).
  const float scale = op->scale().has_value() ? *op->scale() : 1.0f;
  const size_t wsBytes = ttb_sdpa_decode_workspace_bytes(B, H, S, D);
  std::vector<uint32_t> wsShape{static_cast<uint32_t>((wsBytes + 3) / 4)};
  TensorPtr ws = makeDeviceTensor(dev, wsShape, DataType::Float32);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_sdpa_decode(q->shards[i]->ptr, k->shards[i]->ptr, v->shards[i]->ptr, pos ? pos->shards[i]->ptr : nullptr,
                             mask ? mask->shards[i]->ptr : nullptr, out->shards[i]->ptr, ttbDtype(q->dtype), B, H, Hkv, S, D, maskB,
                             maskH, scale, op->is_causal() ? 1 : 0, ws->shards[i]->ptr, wsBytes, r.stream));
  });
  put(op->out(), out);
}

// Paged caches: cache [blocks, heads, block_size, D]; the page table is read on the device.
void Executor::runPagedUpdateCache(const fbt::PagedUpdateCacheOp *op) {
  TensorPtr cache = getDevice(op->cache()), in = getDevice(op->input()), idx = getDevice(op->update_index());
  TensorPtr table = op->page_table() ? getDevice(op->page_table()) : nullptr;
  TTRT_ASSERT(cache->shape.size() == 4 && in->shape.size() == 4 && cache->dtype == in->dtype, "paged_update_cache expects 4-D tensors of one type");
  TTRT_ASSERT(in->shape[2] == cache->shape[1] && in->shape[3] == cache->shape[3], "paged_update_cache input must be [users, seq, heads, head_dim]");
  const size_t users = in->shape[0];
  TTRT_ASSERT(idx->volume() >= users && (idx->dtype == DataType::Int32 || idx->dtype == DataType::UInt32),
              "paged_update_cache needs one Int32 / UInt32 position per user");
  size_t pages = 0;
  if (table) {
    TTRT_ASSERT(table->shape.size() == 2 && table->shape[0] >= users && (table->dtype == DataType::Int32 || table->dtype == DataType::UInt32),
                "page table must be [users, pages] of Int32 / UInt32");
    pages = table->shape[1];
  }
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_paged_update_cache(cache->shards[i]->ptr, in->shards[i]->ptr, idx->shards[i]->ptr, table ? table->shards[i]->ptr : nullptr,
                                    ttbDtype(cache->dtype), ttbDtype(idx->dtype), table ? ttbDtype(table->dtype) : 0, users, in->shape[1],
                                    in->shape[2], cache->shape[0], cache->shape[2], pages, cache->shape[3], r.stream));
  });
  TensorPtr root = cache->base ? cache->base : cache;
  root->version.store(TensorImpl::nextTensorVersion());
}

void Executor::runPagedFillCache(const fbt::PagedFillCacheOp *op) {
  TensorPtr cache = getDevice(op->cache()), in = getDevice(op->input()), table = getDevice(op->page_table());
  TensorPtr bidx = op->batch_idx_tensor() ? getDevice(op->batch_idx_tensor()) : nullptr;
  TTRT_ASSERT(cache->shape.size() == 4 && in->shape.size() == 4 && cache->dtype == in->dtype, "paged_fill_cache expects 4-D tensors of one type");
  TTRT_ASSERT(in->shape[1] == cache->shape[1] && in->shape[3] == cache->shape[3], "paged_fill_cache input must be [users, heads, seq, head_dim]");
  TTRT_ASSERT(table->shape.size() == 2 && (table->dtype == DataType::Int32 || table->dtype == DataType::UInt32),
              "page table must be [rows, pages] of Int32 / UInt32");
  if (bidx) {
    TTRT_ASSERT(bidx->volume() >= in->shape[0] && (bidx->dtype == DataType::Int32 || bidx->dtype == DataType::UInt32),
                "batch index must hold one Int32 / UInt32 per user");
  }
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_paged_fill_cache(cache->shards[i]->ptr, in->shards[i]->ptr, table->shards[i]->ptr, bidx ? bidx->shards[i]->ptr : nullptr,
                                  ttbDtype(cache->dtype), ttbDtype(table->dtype), bidx ? ttbDtype(bidx->dtype) : 0, in->shape[0],
                                  in->shape[1], in->shape[2], cache->shape[0], cache->shape[2], table->shape[0], table->shape[1],
                                  cache->shape[3], r.stream));
  });
  TensorPtr root = cache->base ? cache->base : cache;
  root->version.store(TensorImpl::nextTensorVersion());
}

// q [B, 1, H, D] against paged k, v [blocks, Hkv, block_size, D] (tools/golden/mapping.py:8745-8844).
void Executor::runPagedSdpaDecode(const fbt::PagedScaledDotProductAttentionDecodeOp *op) {
  TTRT_ASSERT(!op->attention_sink(), "attention sinks are not supported");
  TTRT_ASSERT(!op->sliding_window_size().has_value(), "sliding-window decode attention is not supported");
  TensorPtr q = getDevice(op->query()), k = getDevice(op->key()), v = getDevice(op->value());
  TensorPtr table = castOnDevice(getDevice(op->page_table()), DataType::Int32);
  TensorPtr mask = op->attention_mask() ? getDevice(op->attention_mask()) : nullptr;
  TensorPtr pos = op->cur_pos_tensor() ? getDevice(op->cur_pos_tensor()) : nullptr;
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(q->shape.size() == 4 && k->shape.size() == 4 && v->shape == k->shape && q->shape[1] == 1,
              "paged sdpa_decode expects q [B, 1, H, D], k / v [blocks, Hkv, block_size, D]");
  TTRT_ASSERT(q->dtype == k->dtype && q->dtype == v->dtype && out->dtype == q->dtype && out->volume() == q->volume(),
              "paged sdpa_decode operands must share one data type");
  const int B = static_cast<int>(q->shape[0]), H = static_cast<int>(q->shape[2]), D = static_cast<int>(q->shape[3]);
  const int blocks = static_cast<int>(k->shape[0]), Hkv = static_cast<int>(k->shape[1]), blockSize = static_cast<int>(k->shape[2]);
  TTRT_ASSERT(static_cast<int>(k->shape[3]) == D, "paged sdpa_decode operands disagree on head_dim");
  TTRT_ASSERT(table->shape.size() == 2 && static_cast<int>(table->shape[0]) >= B, "page table must be [B, pages]");
  const int pages = static_cast<int>(table->shape[1]), S = pages * blockSize;
  int maskB = 0, maskH = 0;
  if (mask) {
    TTRT_ASSERT(mask->shape.size() == 4 && mask->shape[1] == 1 && static_cast<int>(mask->shape[3]) == S && mask->dtype == q->dtype,
                "paged sdpa_decode mask must be [B or 1, 1, H or 1, pages * block_size] in the operands' data type");
    maskB = static_cast<int>(mask->shape[0]);
    maskH = static_cast<int>(mask->shape[2]);
  }
  if (pos) {
    TTRT_ASSERT(static_cast<int>(pos->volume()) == B && (pos->dtype == DataType::Int32 || pos->dtype == DataType::UInt32),
                "cur_pos must hold one 32-bit integer per user");
  }
  // torch's scaled_dot_product_attention, which the golden calls, scales by 1 / sqrt(D) when no scale is given
  const float scale = op->scale().has_value() ? *op->scale() : 1.0f / std::sqrt(static_cast<float>(D));
  const size_t wsBytes = ttb_sdpa_decode_workspace_bytes(B, H, S, D);
  TensorPtr ws = makeDeviceTensor(dev, {static_cast<uint32_t>((wsBytes + 3) / 4)}, DataType::Float32);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_sdpa_decode_paged(q->shards[i]->ptr, k->shards[i]->ptr, v->shards[i]->ptr, table->shards[i]->ptr,
                                   pos ? pos->shards[i]->ptr : nullptr, mask ? mask->shards[i]->ptr : nullptr, out->shards[i]->ptr,
                                   ttbDtype(q->dtype), B, H, Hkv, blocks, blockSize, pages, D, maskB, maskH, scale,
                                   op->is_causal() ? 1 : 0, ws->shards[i]->ptr, wsBytes, r.stream));
  });
  put(op->out(), out);
}

// ---- indexing ---------------------------------------------------------------------------------------------------
static std::vector<int64_t> shape64(const std::vector<uint32_t> &s) { return std::vector<int64_t>(s.begin(), s.end()); }

void Executor::runGather(const fbt::GatherOp *op) {
  TensorPtr x = getDevice(op->input()), index = getDevice(op->index());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(x->shape.size() == index->shape.size() && !x->shape.empty() && out->shape == index->shape && out->dtype == x->dtype,
              "gather: input and index must have one rank, the result the index's shape");
  const int dim = normDim(op->dim(), x->shape.size());
  std::vector<int64_t> xs = shape64(x->shape), is = shape64(index->shape);
  dev->ranIndexOp = true;
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_gather(x->shards[i]->ptr, index->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(x->dtype), ttbDtype(index->dtype),
                        static_cast<int>(xs.size()), xs.data(), is.data(), dim, r.stream));
  });
  put(op->out(), out);
}

void Executor::runScatter(const fbt::ScatterOp *op) {
  TensorPtr x = getDevice(op->input()), index = getDevice(op->index()), src = getDevice(op->source());
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(x->shape.size() == index->shape.size() && x->shape.size() == src->shape.size() && !x->shape.empty() &&
                  out->shape == x->shape && out->dtype == x->dtype && src->dtype == x->dtype,
              "scatter: input, index and source must have one rank; result and source the input's type");
  const int dim = normDim(op->dim(), x->shape.size());
  std::vector<int64_t> xs = shape64(x->shape), is = shape64(index->shape), ss = shape64(src->shape);
  dev->ranIndexOp = true;
  const int mode = static_cast<int>(op->scatter_reduce_type());
  const size_t wsBytes = ttb_scatter_workspace_bytes(ttbDtype(x->dtype), mode, x->volume());
  TensorPtr ws = wsBytes ? makeDeviceTensor(dev, {static_cast<uint32_t>((wsBytes + 3) / 4)}, DataType::Float32) : nullptr;
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_scatter(x->shards[i]->ptr, index->shards[i]->ptr, src->shards[i]->ptr, out->shards[i]->ptr, ttbDtype(x->dtype),
                         ttbDtype(index->dtype), static_cast<int>(xs.size()), xs.data(), is.data(), ss.data(), dim, mode,
                         ws ? ws->shards[i]->ptr : nullptr, wsBytes, r.stream));
  });
  put(op->out(), out);
}

// The kernel sorts rows; any other dimension is brought to the back with a strided copy first and the
// results are copied back into place.
void Executor::sortAlong(const TensorPtr &x, int dim, bool descending, size_t take, const fbt::TensorRef *valuesRef,
                         const fbt::TensorRef *indicesRef) {
  const size_t rank = x->shape.size();
  TTRT_ASSERT(rank >= 1, "sort of a scalar");
  const size_t n = x->shape[dim];
  TTRT_ASSERT(take <= n, "top-k asks for more entries than the dimension has");
  const bool last = static_cast<size_t>(dim) + 1 == rank;
  // x with `dim` moved to the back (dense)
  TensorPtr rows = x;
  std::vector<uint32_t> movedShape = x->shape;
  std::vector<int64_t> dense = denseStrides(x->shape);
  if (!last) {
    std::vector<int64_t> strides = dense;
    movedShape.erase(movedShape.begin() + dim);
    movedShape.push_back(static_cast<uint32_t>(n));
    strides.erase(strides.begin() + dim);
    strides.push_back(dense[dim]);
    rows = stridedView(x, movedShape, strides, 0, x->dtype);
  }
  const size_t nRows = n ? x->volume() / n : 0;
  TensorPtr values = valuesRef ? allocOut(valuesRef) : nullptr;
  TensorPtr indices = indicesRef ? allocOut(indicesRef) : nullptr;
  std::vector<uint32_t> resShape = movedShape;
  resShape.back() = static_cast<uint32_t>(take);
  TensorPtr v2 = values, i2 = indices;
  if (!last) {
    if (values) v2 = makeDeviceTensor(dev, resShape, values->dtype);
    if (indices) i2 = makeDeviceTensor(dev, resShape, indices->dtype);
  }
  const size_t wsBytes = ttb_sort_workspace_bytes(nRows, n);
  TensorPtr ws = makeDeviceTensor(dev, {static_cast<uint32_t>((wsBytes + 3) / 4)}, DataType::UInt32);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_sort(rows->shards[i]->ptr, v2 ? v2->shards[i]->ptr : nullptr, i2 ? i2->shards[i]->ptr : nullptr, ttbDtype(x->dtype),
                      i2 ? ttbDtype(i2->dtype) : 0, nRows, n, take, descending ? 1 : 0, ws->shards[i]->ptr, wsBytes, r.stream));
  });
  if (!last) {
    // back: result[..., j at `dim`, ...] = moved[..., j]
    std::vector<uint32_t> outShape = x->shape;
    outShape[dim] = static_cast<uint32_t>(take);
    std::vector<int64_t> movedDense = denseStrides(resShape), strides(rank);
    for (size_t d = 0, m = 0; d < rank; ++d) strides[d] = static_cast<int>(d) == dim ? movedDense[rank - 1] : movedDense[m++];
    auto copyBack = [&](const TensorPtr &from, const TensorPtr &to) {
      std::vector<int64_t> shape(outShape.begin(), outShape.end());
      eachRank([&](size_t i, const RankCtx &r) {
        TTB_CALL(ttb_strided_copy(from->shards[i]->ptr, to->shards[i]->ptr, static_cast<int>(dataTypeSize(to->dtype)), static_cast<int>(rank),
                                  shape.data(), strides.data(), 0, r.stream));
      });
    };
    if (values) copyBack(v2, values);
    if (indices) copyBack(i2, indices);
  }
  if (values) put(valuesRef, values);
  if (indices) put(indicesRef, indices);
}

void Executor::runSort(const fbt::SortOp *op) {
  TensorPtr x = getDevice(op->in());
  TTRT_ASSERT(op->outputs() && op->outputs()->size() == 2, "sort produces values and indices");
  const int dim = normDim(op->dim(), x->shape.size());
  sortAlong(x, dim, op->descending(), x->shape[dim], op->outputs()->Get(0), op->outputs()->Get(1)); // always stable
}

void Executor::runTopK(const fbt::TopKOp *op) {
  TensorPtr x = getDevice(op->input_tensor());
  TTRT_ASSERT(op->outputs() && op->outputs()->size() == 2, "top-k produces values and indices");
  TTRT_ASSERT(op->k() >= 0, "negative k");
  const int dim = normDim(op->dim(), x->shape.size());
  sortAlong(x, dim, op->largest(), static_cast<size_t>(op->k()), op->outputs()->Get(0), op->outputs()->Get(1)); // always sorted
}

void Executor::runSampling(const fbt::SamplingOp *op) {
  TensorPtr values = getDevice(op->input_values()), indices = getDevice(op->input_indices());
  TensorPtr k = castOnDevice(getDevice(op->k()), DataType::UInt32);
  TensorPtr p = castOnDevice(getDevice(op->p()), values->dtype), temp = castOnDevice(getDevice(op->temp()), values->dtype);
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(values->shape.size() >= 2 && values->shape == indices->shape, "sampling: values and indices must be [.., batch, candidates]");
  const size_t candidates = values->shape.back(), rows = values->volume() / std::max<size_t>(candidates, 1);
  TTRT_ASSERT(out->volume() == rows && k->volume() == rows && p->volume() == rows && temp->volume() == rows,
              "sampling: k, p, temp and the result hold one entry per row");
  // Without a seed every call draws differently: a process-wide counter stands in for the device RNG state.
  static std::atomic<uint64_t> unseeded{0x5eed};
  const uint64_t seed = op->seed().has_value() ? *op->seed() : unseeded.fetch_add(0x9E3779B97F4A7C15ull);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_sampling(values->shards[i]->ptr, indices->shards[i]->ptr, k->shards[i]->ptr, p->shards[i]->ptr, temp->shards[i]->ptr,
                          out->shards[i]->ptr, ttbDtype(values->dtype), ttbDtype(indices->dtype), ttbDtype(out->dtype),
                          static_cast<int>(rows), static_cast<int>(candidates), seed, r.stream));
  });
  put(op->out(), out);
}

// ---- data movement --------------------------------------------------------------------------------------------
void Executor::runReshape(const fbt::ReshapeOp *op) {
  TensorPtr in = get(op->in());
  std::vector<uint32_t> shape = refShape(op->out());
  TTRT_ASSERT(prod(shape, 0, shape.size()) == in->volume(), "reshape changes the element count");
  // Dense row-major on both sides: a reshape is a new view of the same memory.
  auto view = std::make_shared<TensorImpl>();
  view->shape = shape;
  view->stride = denseStrides(shape);
  view->dtype = in->dtype;
  view->storage = in->storage;
  view->layout = in->layout;
  view->shards = in->shards;
  view->device = in->device;
  put(op->out(), view);
}

TensorPtr Executor::stridedView(const TensorPtr &in, const std::vector<uint32_t> &outShape, const std::vector<int64_t> &inStrides,
                                int64_t offset, DataType dt) {
  TensorPtr out = makeDeviceTensor(dev, outShape, dt);
  out->layout = in->layout;
  std::vector<int64_t> shape(outShape.begin(), outShape.end());
  TTRT_ASSERT(shape.size() <= 8, "rank above 8");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_strided_copy(in->shards[i]->ptr, out->shards[i]->ptr, static_cast<int>(dataTypeSize(dt)),
                              static_cast<int>(shape.size()), shape.data(), inStrides.data(), offset, r.stream));
  });
  return out;
}

void Executor::runPermute(const fbt::TensorRef *inRef, const std::vector<int> &perm, const fbt::TensorRef *outRef) {
  TensorPtr in = getDevice(inRef);
  size_t rank = in->shape.size();
  TTRT_ASSERT(perm.size() == rank, "permutation rank mismatch");
  std::vector<uint32_t> outShape(rank);
  std::vector<int64_t> strides(rank);
  std::vector<int64_t> dense = denseStrides(in->shape);
  for (size_t k = 0; k < rank; ++k) {
    int p = normDim(perm[k], rank);
    outShape[k] = in->shape[p]; // TTNN permute: outputDim[i] = inputDim[permutation[i]]
    strides[k] = dense[p];
  }
  TTRT_ASSERT(outShape == refShape(outRef), "permute result shape differs from the op's result type");
  if (fuse && rank == 4 && strides[3] == 1 && singleUse(outRef)) {
    auto use = info.firstUse.find(outRef->global_id());
    if (use != info.firstUse.end()) {
      const auto *consumer = prog->operations()->Get(use->second);
      bool strided = false;
      if (consumer->type_type() == OpType::RotaryEmbeddingOp) {
        strided = consumer->type_as_RotaryEmbeddingOp()->input()->global_id() == outRef->global_id();
      } else if (consumer->type_type() == OpType::ScaledDotProductAttentionOp) {
        const auto *a = consumer->type_as_ScaledDotProductAttentionOp();
        strided = !a->attention_mask() && !a->attention_sink();
      }
      if (strided) {
        lazy[outRef->global_id()] = LazyView{in, outShape, strides};
        return;
      }
    }
  }
  put(outRef, stridedView(in, outShape, strides, 0, in->dtype));
}

void Executor::runConcat(const fbt::ConcatOp *op) {
  TTRT_ASSERT(op->inputs() && op->inputs()->size() > 0, "concat without inputs");
  TensorPtr out = allocOut(op->out());
  size_t rank = out->shape.size();
  int d = normDim(op->dim(), rank);
  std::vector<int64_t> outStrides = denseStrides(out->shape);
  int64_t at = 0;
  for (const auto *ref : *op->inputs()) {
    TensorPtr in = getDevice(ref);
    TTRT_ASSERT(in->shape.size() == rank && in->dtype == out->dtype, "concat inputs must match in rank and data type");
    std::vector<int64_t> shape(in->shape.begin(), in->shape.end());
    int64_t offset = at * outStrides[d];
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_strided_scatter(in->shards[i]->ptr, out->shards[i]->ptr, static_cast<int>(dataTypeSize(in->dtype)),
                                   static_cast<int>(rank), shape.data(), outStrides.data(), offset, r.stream));
    });
    at += in->shape[d];
  }
  TTRT_ASSERT(at == out->shape[d], "concat inputs do not add up to the result extent");
  put(op->out(), out);
}

void Executor::runSlice(const fbt::SliceOp *op) {
  TensorPtr in = getDevice(op->in());
  const auto *p = op->params_as_SliceStaticOpParams();
  TTRT_ASSERT(p && p->begins() && p->ends(), "only static slices are supported");
  size_t rank = in->shape.size();
  TTRT_ASSERT(p->begins()->size() == rank && p->ends()->size() == rank, "slice bounds rank mismatch");
  std::vector<int64_t> dense = denseStrides(in->shape), strides(rank);
  std::vector<uint32_t> outShape(rank);
  int64_t offset = 0;
  for (size_t k = 0; k < rank; ++k) {
    int64_t b = p->begins()->Get(static_cast<uint32_t>(k)), e = p->ends()->Get(static_cast<uint32_t>(k));
    int64_t st = op->step() && op->step()->size() == rank ? op->step()->Get(static_cast<uint32_t>(k)) : 1;
    int64_t dim = in->shape[k];
    if (b < 0) b += dim;
    if (e < 0) e += dim;
    TTRT_ASSERT(st > 0 && b >= 0 && e <= dim && b <= e, "slice bounds out of range on dim ", k);
    outShape[k] = static_cast<uint32_t>((e - b + st - 1) / st);
    strides[k] = dense[k] * st;
    offset += b * dense[k];
  }
  TTRT_ASSERT(outShape == refShape(op->out()), "slice result shape differs from the op's result type");
  put(op->out(), stridedView(in, outShape, strides, offset, in->dtype));
}

void Executor::runRepeat(const fbt::RepeatOp *op) {
  TensorPtr in = getDevice(op->in());
  size_t rank = in->shape.size();
  TTRT_ASSERT(op->repeat_dims() && op->repeat_dims()->size() == rank, "repeat dims rank mismatch");
  // out[i] = in[i mod shape]: view each dim as (repeat, size) with stride (0, dense)
  std::vector<uint32_t> viewShape;
  std::vector<int64_t> viewStrides, dense = denseStrides(in->shape);
  for (size_t k = 0; k < rank; ++k) {
    viewShape.push_back(static_cast<uint32_t>(op->repeat_dims()->Get(static_cast<uint32_t>(k))));
    viewStrides.push_back(0);
    viewShape.push_back(in->shape[k]);
    viewStrides.push_back(dense[k]);
  }
  TTRT_ASSERT(viewShape.size() <= 8, "repeat of rank above 4 is not supported");
  TensorPtr t = stridedView(in, viewShape, viewStrides, 0, in->dtype);
  t->shape = refShape(op->out());
  t->stride = denseStrides(t->shape);
  TTRT_ASSERT(t->volume() == prod(viewShape, 0, viewShape.size()), "repeat result shape differs from the op's result type");
  put(op->out(), t);
}

void Executor::runRepeatInterleave(const fbt::RepeatInterleaveOp *op) {
  TensorPtr in = getDevice(op->input());
  size_t rank = in->shape.size();
  int d = normDim(op->dim(), rank);
  std::vector<uint32_t> viewShape;
  std::vector<int64_t> viewStrides, dense = denseStrides(in->shape);
  for (size_t k = 0; k < rank; ++k) {
    viewShape.push_back(in->shape[k]);
    viewStrides.push_back(dense[k]);
    if (static_cast<int>(k) == d) {
      viewShape.push_back(op->repeats());
      viewStrides.push_back(0);
    }
  }
  TTRT_ASSERT(viewShape.size() <= 8, "rank above 7");
  TensorPtr t = stridedView(in, viewShape, viewStrides, 0, in->dtype);
  t->shape = refShape(op->out());
  t->stride = denseStrides(t->shape);
  TTRT_ASSERT(t->volume() == prod(viewShape, 0, viewShape.size()), "repeat_interleave result shape differs from the op's result type");
  put(op->out(), t);
}

// [B, H, S, D] -> [B, S, H*D]
void Executor::runConcatenateHeads(const fbt::ConcatenateHeadsOp *op) {
  TensorPtr in = getDevice(op->in());
  TTRT_ASSERT(in->shape.size() == 4, "concatenate_heads expects [batch, heads, seq, head_dim]");
  uint32_t B = in->shape[0], H = in->shape[1], S = in->shape[2], D = in->shape[3];
  std::vector<int64_t> dense = denseStrides(in->shape);
  TensorPtr t = stridedView(in, {B, S, H, D}, {dense[0], dense[2], dense[1], dense[3]}, 0, in->dtype);
  t->shape = {B, S, H * D};
  t->stride = denseStrides(t->shape);
  TTRT_ASSERT(t->shape == refShape(op->out()), "concatenate_heads result shape differs from the op's result type");
  put(op->out(), t);
}

// Fused [B, S, (Hq + 2*Hkv)*D] (or q and packed kv) -> q [B,Hq,S,D], k [B,Hkv,S,D] (or [B,Hkv,D,S]), v [B,Hkv,S,D]
// Semantics: tools/tt-alchemist/templates/python/local/ttir_cpu.py:824-864.
void Executor::runSplitQkv(const fbt::SplitQueryKeyValueAndSplitHeadsOp *op) {
  TensorPtr in = getDevice(op->in());
  TensorPtr kv = op->kv_input() ? getDevice(op->kv_input()) : nullptr;
  TTRT_ASSERT(in->shape.size() == 3, "split_query_key_value_and_split_heads expects [batch, seq, hidden]");
  uint32_t B = in->shape[0], S = in->shape[1], hidden = in->shape[2];
  uint32_t Hq = op->num_heads(), Hkv = op->num_kv_heads().value_or(Hq);
  uint32_t D = kv ? hidden / Hq : hidden / (Hq + 2 * Hkv);
  auto heads = [&](const TensorPtr &src, uint32_t rowLen, uint32_t colOff, uint32_t H, bool transpose) {
    // element (b, h, s, d) = src[b, s, colOff + h*D + d]
    int64_t sb = static_cast<int64_t>(S) * rowLen, ss = rowLen;
    if (!transpose) {
      return stridedView(src, {B, H, S, D}, {sb, static_cast<int64_t>(D), ss, 1}, colOff, src->dtype);
    }
    return stridedView(src, {B, H, D, S}, {sb, static_cast<int64_t>(D), 1, ss}, colOff, src->dtype);
  };
  TensorPtr q, k, v;
  if (!kv) {
    q = heads(in, hidden, 0, Hq, false);
    k = heads(in, hidden, Hq * D, Hkv, op->transpose_key());
    v = heads(in, hidden, (Hq + Hkv) * D, Hkv, false);
  } else {
    TTRT_ASSERT(kv->shape.size() == 3 && kv->shape[2] == 2 * Hkv * D, "kv input must be [batch, seq, 2*kv_heads*head_dim]");
    q = heads(in, hidden, 0, Hq, false);
    k = heads(kv, kv->shape[2], 0, Hkv, op->transpose_key());
    v = heads(kv, kv->shape[2], Hkv * D, Hkv, false);
  }
  put(op->q_out(), q);
  put(op->k_out(), k);
  put(op->v_out(), v);
}

void Executor::runRotaryEmbedding(const fbt::RotaryEmbeddingOp *op) {
  if (ropeApplied.erase(op->input()->global_id())) {
    // The projection that produced the input stored it rotated: the result is the input (still a pending view).
    auto lz = lazy.find(op->input()->global_id());
    if (lz != lazy.end()) {
      LazyView v = std::move(lz->second);
      lazy.erase(lz);
      lazy[op->out()->global_id()] = std::move(v);
    } else {
      put(op->out(), getDevice(op->input()));
    }
    return;
  }
  TensorPtr c = getDevice(op->cos_cache()), s = getDevice(op->sin_cache());
  std::vector<uint32_t> xs = refShape(op->input());
  TTRT_ASSERT(xs.size() >= 2, "rotary_embedding expects [..., seq, head_dim]");
  size_t rank = xs.size();
  size_t D = xs[rank - 1], S = xs[rank - 2];
  // A pending head split is read through its strides when they are vector-aligned.
  TensorPtr x;
  size_t B = 1, H = 0;
  int64_t strides[3];
  auto lz = lazy.find(op->input()->global_id());
  if (lz != lazy.end() && rank == 4 && lz->second.strides[3] == 1) {
    size_t unit = 16 / dataTypeSize(lz->second.base->dtype);
    const auto &st = lz->second.strides;
    if (st[0] % unit == 0 && st[1] % unit == 0 && st[2] % unit == 0) {
      x = lz->second.base;
      B = xs[0];
      H = xs[1];
      strides[0] = st[0]; strides[1] = st[1]; strides[2] = st[2];
    }
  }
  if (!x) {
    x = getDevice(op->input());
    H = x->volume() / std::max<size_t>(S * D, 1);
    strides[0] = static_cast<int64_t>(H * S * D); strides[1] = static_cast<int64_t>(S * D); strides[2] = static_cast<int64_t>(D);
  }
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(!op->token_index().has_value(), "rotary_embedding with token_index (decode) is not supported");
  TTRT_ASSERT(c->volume() == S * D && s->volume() == S * D, "cos/sin caches must be [seq, head_dim] = [", S, ", ", D, "]");
  TTRT_ASSERT(c->dtype == x->dtype && s->dtype == x->dtype && out->dtype == x->dtype, "rotary_embedding tensors must share one data type");
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_rotary_embedding_strided(x->shards[i]->ptr, c->shards[i]->ptr, s->shards[i]->ptr, out->shards[i]->ptr,
                                          ttbDtype(x->dtype), B, H, S, D, strides, r.stream));
  });
  put(op->out(), out);
}

// Attention with its operands read through strides (pending head splits) and, when the next op
// is concatenate_heads on its result, the output written straight in [batch, seq, heads*dim].
size_t Executor::trySdpa(size_t i) {
  const auto *ops = prog->operations();
  const auto *op = ops->Get(static_cast<uint32_t>(i))->type_as_ScaledDotProductAttentionOp();
  if (op->attention_mask() || op->attention_sink() || op->sliding_window_size().has_value()) return 0;
  std::vector<uint32_t> qs = refShape(op->query()), ks = refShape(op->key()), vs = refShape(op->value());
  DataType dt = refDtype(op->query());
  if (qs.size() != 4 || ks.size() != 4 || vs != ks || qs[3] != 128 || ks[3] != 128 || qs[0] != ks[0] || ks[1] == 0 ||
      qs[1] % ks[1] != 0 || (dt != DataType::BFloat16 && dt != DataType::Float16) || refDtype(op->key()) != dt ||
      refDtype(op->value()) != dt || refDtype(op->out()) != dt || refShape(op->out()) != qs)
    return 0;
  int64_t B = qs[0], Hq = qs[1], Sq = qs[2], D = qs[3], Hkv = ks[1], Skv = ks[2];
  // next op: concatenate_heads of the (single-use) result?
  std::vector<const fbt::Operation *> deallocs;
  size_t j = i + 1;
  const auto *nop = peek(j, deallocs);
  const fbt::ConcatenateHeadsOp *merge = nullptr;
  if (nop && nop->type_type() == OpType::ConcatenateHeadsOp && singleUse(op->out())) {
    const auto *m = nop->type_as_ConcatenateHeadsOp();
    std::vector<uint32_t> want = {qs[0], qs[2], qs[1] * qs[3]};
    if (m->in()->global_id() == op->out()->global_id() && refShape(m->out()) == want && refDtype(m->out()) == dt) merge = m;
  }
  bool anyLazy = lazy.count(op->query()->global_id()) || lazy.count(op->key()->global_id()) || lazy.count(op->value()->global_id());
  if (!merge && !anyLazy) return 0;
  auto q = viewOf(op->query()), k = viewOf(op->key()), v = viewOf(op->value());
  for (const auto *pv : {&q, &k, &v}) {
    for (int d = 0; d < 3; ++d) {
      if (pv->second[d] % 8 != 0) return 0; // get() will materialise in the plain path
    }
    if (pv->second[3] != 1) return 0;
  }
  const fbt::TensorRef *outRef = merge ? merge->out() : op->out();
  TensorPtr out = allocOut(outRef);
  int64_t os[3];
  if (merge) { os[0] = Sq * Hq * D; os[1] = D; os[2] = Hq * D; }
  else { os[0] = Hq * Sq * D; os[1] = Sq * D; os[2] = D; }
  float scale = op->scale().value_or(1.0f / std::sqrt(static_cast<float>(D)));
  bool unsupported = false;
  eachRank([&](size_t r, const RankCtx &rc) {
    if (unsupported) return;
    int st = ttb_sdpa_strided(q.first->shards[r]->ptr, k.first->shards[r]->ptr, v.first->shards[r]->ptr, out->shards[r]->ptr,
                              ttbDtype(dt), B, Hq, Hkv, Sq, Skv, D, q.second.data(), k.second.data(), v.second.data(), os,
                              op->is_causal() ? 1 : 0, scale, rc.stream);
    if (st == TTB_ERR_UNSUPPORTED && r == 0) unsupported = true;
    else TTB_CALL(st);
  });
  if (unsupported) return 0; // nothing was launched; the plain path copies the views and runs dense
  put(outRef, out);
  if (!merge) return 1;
  runDeallocs(deallocs);
  return j + 1 - i;
}

void Executor::runSdpa(const fbt::ScaledDotProductAttentionOp *op) {
  TensorPtr q = getDevice(op->query()), k = getDevice(op->key()), v = getDevice(op->value());
  TensorPtr mask = op->attention_mask() ? getDevice(op->attention_mask()) : nullptr;
  TTRT_ASSERT(!op->attention_sink(), "attention_sink is not supported");
  TTRT_ASSERT(!op->sliding_window_size().has_value(), "sliding_window_size is not supported");
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(q->shape.size() == 4 && k->shape.size() == 4 && v->shape.size() == 4, "attention operands must be [batch, heads, seq, head_dim]");
  int64_t B = q->shape[0], Hq = q->shape[1], Sq = q->shape[2], D = q->shape[3];
  int64_t Hkv = k->shape[1], Skv = k->shape[2];
  TTRT_ASSERT(k->shape[0] == B && v->shape[0] == B && k->shape[3] == D && v->shape == k->shape, "attention operand shapes disagree");
  TTRT_ASSERT(Hkv > 0 && Hq % Hkv == 0, "query heads must be a multiple of key/value heads");
  TTRT_ASSERT(q->dtype == k->dtype && q->dtype == v->dtype && q->dtype == out->dtype, "attention tensors must share one data type");
  float scale = op->scale().value_or(1.0f / std::sqrt(static_cast<float>(D)));
  int64_t mb = 0, mh = 0;
  if (mask) {
    TTRT_ASSERT(mask->shape.size() == 4 && mask->shape[2] == Sq && mask->shape[3] == Skv && mask->dtype == q->dtype,
                "attention mask must be [1|B, 1|H, Sq, Skv] in the operand data type");
    mb = mask->shape[0];
    mh = mask->shape[1];
  }
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_sdpa(q->shards[i]->ptr, k->shards[i]->ptr, v->shards[i]->ptr, mask ? mask->shards[i]->ptr : nullptr,
                      out->shards[i]->ptr, ttbDtype(q->dtype), B, Hq, Hkv, Sq, Skv, D, mb, mh, op->is_causal() ? 1 : 0, scale,
                      r.stream));
  });
  put(op->out(), out);
}

// ---- mesh ops -------------------------------------------------------------------------------------------------
uint32_t Executor::meshAxisSize(uint32_t clusterAxis) const {
  TTRT_ASSERT(clusterAxis < 2, "cluster_axis must be 0 or 1");
  return dev->meshShape[clusterAxis];
}

// The peer-memory all-reduce needs one workspace per rank that every other rank has mapped.
// They are set up at the first all-reduce of a device (a collective step: every rank gets here
// with the same program).  TTB_DISABLE_SYMM_AR=1, or any failure to map a peer, leaves NCCL in
// charge.
bool Executor::symmReady(size_t bytes) {
  static const bool disabled = [] {
    const char *e = std::getenv("TTB_DISABLE_SYMM_AR");
    return e && e[0] == '1';
  }();
  if (disabled) return false;
  if (!dev->symmTried) {
    dev->symmTried = true;
    constexpr size_t kMaxOperand = size_t(64) << 20;
    int rc;
    if (dev->multiProcess) {
      RankCtx &r = dev->locals[0];
      TTB_CALL(ttb_set_device(r.cudaDevice));
      rc = ttb_symm_create_rank(&r.symm, r.comm, static_cast<int>(r.meshRank), static_cast<int>(dev->worldSize), kMaxOperand,
                                r.stream);
    } else {
      std::vector<void *> symms(dev->locals.size(), nullptr);
      std::vector<int> ids;
      for (const RankCtx &r : dev->locals) ids.push_back(r.cudaDevice);
      rc = ttb_symm_create_all(symms.data(), static_cast<int>(ids.size()), ids.data(), kMaxOperand);
      if (rc == TTB_OK) {
        for (size_t i = 0; i < symms.size(); ++i) dev->locals[i].symm = symms[i];
      }
    }
    if (rc != TTB_OK) logDebug(std::string("peer-memory all-reduce unavailable, using NCCL: ") + ttb_last_error());
  }
  for (const RankCtx &r : dev->locals) {
    if (!r.symm || bytes > ttb_symm_max_bytes(r.symm)) return false;
  }
  return true;
}

// A tensor whose only consumer is the next all-reduce (a sum over a float type, no other
// all-reduce in between) is produced straight into the staging region of that all-reduce, which
// then has nothing to copy.
bool Executor::feedsSymmAllReduce(const fbt::TensorRef *ref) {
  if (!fuse || dev->worldSize == 1 || !singleUse(ref)) return false;
  auto use = info.firstUse.find(ref->global_id());
  if (use == info.firstUse.end() || use->second <= curOp) return false;
  const auto *ops = prog->operations();
  const auto *consumer = ops->Get(use->second);
  if (consumer->type_type() != OpType::AllReduceOp) return false;
  const auto *ar = consumer->type_as_AllReduceOp();
  if (static_cast<int>(ar->reduce_type()) != 0 || meshAxisSize(ar->cluster_axis()) == 1) return false;
  for (uint32_t k = static_cast<uint32_t>(curOp) + 1; k < use->second; ++k) {
    if (ops->Get(k)->type_type() == OpType::AllReduceOp) return false;
  }
  DataType dt = refDtype(ref);
  return dt == DataType::BFloat16 || dt == DataType::Float16 || dt == DataType::Float32;
}

// The row-parallel projections of a tensor-parallel block (o_proj, down_proj) produce partial sums
// that only the following all-reduce reads.  Their GEMM stores every row block of its result from
// the epilogue into the workspace of the rank that reduces that block, so the reduce-scatter half
// of the all-reduce has happened by the time the GEMM ends.  TTB_DISABLE_GEMM_PUSH=1 turns it off.
TensorPtr Executor::tryGemmPush(const TensorPtr &a, const TensorPtr &b, const fbt::TensorRef *outRef, int64_t M, int64_t N,
                                int64_t K) {
  static const bool disabled = [] {
    const char *e = std::getenv("TTB_DISABLE_GEMM_PUSH");
    return e && e[0] == '1';
  }();
  if (disabled || !feedsSymmAllReduce(outRef)) return nullptr;
  DataType dt = refDtype(outRef);
  if ((dt != DataType::BFloat16 && dt != DataType::Float16) || a->dtype != dt) return nullptr;
  const int64_t n = dev->worldSize;
  const size_t bytes = static_cast<size_t>(M) * N * dataTypeSize(dt);
  if (M % n != 0 || (M / n) % 128 != 0 || bytes % (16 * n) != 0 || !symmReady(bytes)) return nullptr;
  // Everything that decides between this path and the ordinary one must be the same on every rank
  // (ranks may be separate processes, and a rank that produced an ordinary tensor while its peers
  // pushed would be summed from the wrong regions).  So the shape rules of the tensor-core kernel and
  // the switch that disables it are checked here, from facts all ranks share, and a refusal for any
  // other reason (an operand that is not 16-byte aligned on one rank) is an error, not a fallback.
  static const bool tensorCoreOff = [] {
    const char *e = std::getenv("TTB_DISABLE_TCGEN05");
    return e && e[0] && std::strcmp(e, "0") != 0;
  }();
  if (tensorCoreOff || K % 8 != 0 || K < 8 || N < 8 || (N * static_cast<int64_t>(dataTypeSize(dt))) % 16 != 0 ||
      M * N * K < (1ll << 18) || M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff)
    return nullptr;
  auto t = std::make_shared<TensorImpl>();
  t->shape = refShape(outRef);
  t->stride = denseStrides(t->shape);
  t->dtype = dt;
  t->storage = Storage::Device;
  t->layout = refLayout(outRef);
  t->device = dev;
  t->pushedForAllReduce = true;
  eachRank([&](size_t i, const RankCtx &r) {
    void *targets[8] = {};
    int rank = 0, nranks = 0;
    TTB_CALL(ttb_symm_push_targets(r.symm, bytes, targets, &rank, &nranks));
    int rc = ttb_gemm_push(a->shards[i]->ptr, b->shards[i]->ptr, targets, nranks, ttbDtype(dt), M, N, K, r.stream);
    if (rc != TTB_OK) {
      TTRT_FATAL("ttb_gemm_push failed (", rc, ") on mesh coordinate ", r.meshRank, ": ", ttb_last_error(),
                 " -- the other ranks may already have taken the pushed path, so there is no falling back");
    }
    auto buf = std::make_shared<Buffer>();
    TTB_CALL(ttb_symm_input_buffer(r.symm, bytes, &buf->ptr)); // the region the partials land in; never read as a matrix
    buf->bytes = bytes;
    buf->cudaDevice = r.cudaDevice;
    buf->kind = Buffer::Kind::Borrowed;
    t->shards.push_back(buf);
  });
  return t;
}

TensorPtr Executor::allocForAllReduce(const fbt::TensorRef *ref) {
  if (!feedsSymmAllReduce(ref)) return nullptr;
  DataType dt = refDtype(ref);
  auto t = std::make_shared<TensorImpl>();
  t->shape = refShape(ref);
  t->stride = denseStrides(t->shape);
  t->dtype = dt;
  t->storage = Storage::Device;
  t->layout = refLayout(ref);
  t->device = dev;
  size_t bytes = t->bytes();
  if (bytes == 0 || bytes % 16 != 0 || !symmReady(bytes)) return nullptr;
  for (const RankCtx &r : dev->locals) {
    auto b = std::make_shared<Buffer>();
    TTB_CALL(ttb_symm_input_buffer(r.symm, bytes, &b->ptr));
    b->bytes = bytes;
    b->cudaDevice = r.cudaDevice;
    b->kind = Buffer::Kind::Borrowed; // the workspace owns the memory
    t->shards.push_back(b);
  }
  return t;
}

// out = all_reduce(in) [+ residual].  Sums of float tensors go through the peer-memory kernel
// (one launch per rank, the residual add included); everything else through NCCL, with the add
// as its own launch.
void Executor::allReduce(const TensorPtr &in, const TensorPtr &residual, const TensorPtr &out, int reduceType) {
  // The peer-memory kernel numbers its launches (a replayed launch would repeat a number its
  // peers have moved past), so collectives stay outside traces.
  refuseWhileRecording("a collective");
  bool isFloat = in->dtype == DataType::BFloat16 || in->dtype == DataType::Float16 || in->dtype == DataType::Float32;
  if (in->pushedForAllReduce) {
    TTRT_ASSERT(reduceType == 0, "a scattered GEMM result can only be summed");
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_symm_all_reduce_pushed(r.symm, residual ? residual->shards[i]->ptr : nullptr, out->shards[i]->ptr,
                                          in->volume(), ttbDtype(in->dtype), r.stream));
    });
    return;
  }
  if (reduceType == 0 && isFloat && in->bytes() % 16 == 0 && symmReady(in->bytes())) {
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_symm_all_reduce(r.symm, in->shards[i]->ptr, residual ? residual->shards[i]->ptr : nullptr,
                                   out->shards[i]->ptr, in->volume(), ttbDtype(in->dtype), r.stream));
    });
    return;
  }
  if (dev->locals.size() > 1) TTB_CALL(ttb_group_start());
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_all_reduce(r.comm, in->shards[i]->ptr, out->shards[i]->ptr, in->volume(), ttbDtype(in->dtype), reduceType,
                            r.stream));
  });
  if (dev->locals.size() > 1) TTB_CALL(ttb_group_end());
  if (residual) {
    int64_t shape[1] = {static_cast<int64_t>(out->volume())}, ones[1] = {1};
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_eltwise_binary(static_cast<int>(fbt::EltwiseBinaryOpType::Add), out->shards[i]->ptr, ttbDtype(out->dtype),
                                  residual->shards[i]->ptr, ttbDtype(residual->dtype), out->shards[i]->ptr, ttbDtype(out->dtype),
                                  1, shape, ones, ones, r.stream));
    });
  }
}

void Executor::runAllReduce(const fbt::AllReduceOp *op) {
  TensorPtr in = getDevice(op->in());
  uint32_t n = meshAxisSize(op->cluster_axis());
  if (n == 1) {
    put(op->out(), in);
    return;
  }
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(out->volume() == in->volume() && out->dtype == in->dtype, "all_reduce changes shape or type");
  allReduce(in, nullptr, out, static_cast<int>(op->reduce_type()));
  put(op->out(), out);
}

// all_reduce -> add(x, result) with the result single-use: the residual add rides in the
// all-reduce kernel (both roundings kept).
size_t Executor::tryAllReduceAdd(size_t i) {
  const auto *ops = prog->operations();
  const auto *op = ops->Get(static_cast<uint32_t>(i))->type_as_AllReduceOp();
  if (meshAxisSize(op->cluster_axis()) == 1 || static_cast<int>(op->reduce_type()) != 0 || !singleUse(op->out())) return 0;
  std::vector<const fbt::Operation *> deallocs;
  size_t j = i + 1;
  const auto *nop = peek(j, deallocs);
  if (!nop || nop->type_type() != OpType::EltwiseBinaryOp) return 0;
  const auto *add = nop->type_as_EltwiseBinaryOp();
  if (add->type() != fbt::EltwiseBinaryOpType::Add) return 0;
  const fbt::TensorRef *other = nullptr;
  uint32_t cur = op->out()->global_id();
  if (add->lhs()->global_id() == cur) other = add->rhs();
  else if (add->rhs()->global_id() == cur) other = add->lhs();
  DataType dt = refDtype(op->out());
  if (!other || other->global_id() == cur || refShape(other) != refShape(op->out()) || refDtype(other) != dt ||
      refShape(add->out()) != refShape(op->out()) || refDtype(add->out()) != dt || !pool.count(other->global_id()) ||
      (dt != DataType::BFloat16 && dt != DataType::Float16 && dt != DataType::Float32))
    return 0;
  TensorPtr in = getDevice(op->in()), res = getDevice(other);
  if (in->dtype != dt || in->volume() != res->volume()) return 0;
  // all_reduce -> add -> mesh_partition along the same mesh axis, the sum read by nothing else: every rank keeps
  // only its own block of rows, so the broadcast half of the all-reduce would be thrown away.  The kernel then
  // stops after the reduce-scatter half and writes the partition's result directly.
  static const bool scatterOff = [] {
    const char *e = std::getenv("TTB_DISABLE_REDUCE_SCATTER_FUSION");
    return e && e[0] == '1';
  }();
  if (!scatterOff && singleUse(add->out())) {
    std::vector<const fbt::Operation *> d2;
    size_t j2 = j + 1;
    const auto *pop = peek(j2, d2);
    if (pop && pop->type_type() == OpType::MeshPartitionOp) {
      const auto *part = pop->type_as_MeshPartitionOp();
      const uint32_t n = meshAxisSize(op->cluster_axis());
      const uint32_t axis = part->cluster_axis().value_or(dev->meshShape[0] > 1 ? 0 : 1);
      std::vector<uint32_t> shape = refShape(add->out());
      const int d = normDim(part->dim(), shape.size());
      const bool symm = in->pushedForAllReduce || (in->bytes() % 16 == 0 && symmReady(in->bytes()));
      if (part->in()->global_id() == add->out()->global_id() && axis == op->cluster_axis() && n == dev->worldSize && symm &&
          prod(shape, 0, d) == 1 && shape[d] % n == 0 && (in->bytes() / n) % 16 == 0 && refDtype(part->out()) == dt) {
        refuseWhileRecording("a collective");
        TensorPtr out = allocOut(part->out());
        TTRT_ASSERT(out->volume() * n == in->volume(), "mesh_partition result must be 1/", n, " of its input");
        eachRank([&](size_t r, const RankCtx &rc) {
          if (in->pushedForAllReduce) {
            TTB_CALL(ttb_symm_reduce_scatter_pushed(rc.symm, res->shards[r]->ptr, out->shards[r]->ptr, in->volume(), ttbDtype(dt),
                                                    rc.stream));
          } else {
            TTB_CALL(ttb_symm_reduce_scatter(rc.symm, in->shards[r]->ptr, res->shards[r]->ptr, out->shards[r]->ptr, in->volume(),
                                             ttbDtype(dt), rc.stream));
          }
        });
        put(part->out(), out);
        deallocs.insert(deallocs.end(), d2.begin(), d2.end());
        runDeallocs(deallocs);
        return j2 + 1 - i;
      }
    }
  }
  TensorPtr out = allocOut(add->out());
  allReduce(in, res, out, 0);
  put(add->out(), out);
  runDeallocs(deallocs);
  return j + 1 - i;
}

void Executor::runAllGather(const fbt::AllGatherOp *op) {
  TensorPtr in = getDevice(op->in());
  uint32_t n = meshAxisSize(op->cluster_axis());
  if (n == 1) {
    put(op->out(), in);
    return;
  }
  refuseWhileRecording("a collective");
  size_t rank = in->shape.size();
  int d = normDim(op->all_gather_dim(), rank);
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(out->volume() == in->volume() * n, "all_gather result must be ", n, " times the input");
  size_t outer = prod(in->shape, 0, d);
  // NCCL concatenates rank blocks; that is the result itself when nothing precedes the gather dim.
  TensorPtr staged = outer == 1 ? out : makeDeviceTensor(dev, {n, static_cast<uint32_t>(in->volume())}, in->dtype);
  if (dev->locals.size() > 1) TTB_CALL(ttb_group_start());
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_all_gather(r.comm, in->shards[i]->ptr, staged->shards[i]->ptr, in->volume(), ttbDtype(in->dtype), r.stream));
  });
  if (dev->locals.size() > 1) TTB_CALL(ttb_group_end());
  if (outer != 1) {
    // staged is [n, outer, len, inner]; result is [outer, n*len, inner]
    int64_t len = in->shape[d], inner = static_cast<int64_t>(prod(in->shape, d + 1, rank));
    std::vector<int64_t> shape = {static_cast<int64_t>(outer), static_cast<int64_t>(n), len * inner};
    std::vector<int64_t> strides = {len * inner, static_cast<int64_t>(in->volume()), 1};
    eachRank([&](size_t i, const RankCtx &r) {
      TTB_CALL(ttb_strided_copy(staged->shards[i]->ptr, out->shards[i]->ptr, static_cast<int>(dataTypeSize(in->dtype)), 3,
                                shape.data(), strides.data(), 0, r.stream));
    });
  }
  put(op->out(), out);
}

void Executor::runReduceScatter(const fbt::ReduceScatterOp *op) {
  TensorPtr in = getDevice(op->in());
  uint32_t n = meshAxisSize(op->cluster_axis());
  if (n == 1) {
    put(op->out(), in);
    return;
  }
  refuseWhileRecording("a collective");
  size_t rank = in->shape.size();
  int d = normDim(op->scatter_dim(), rank);
  TensorPtr out = allocOut(op->out());
  TTRT_ASSERT(in->shape[d] % n == 0 && out->volume() * n == in->volume(), "scatter dimension must divide by the mesh axis size");
  size_t outer = prod(in->shape, 0, d);
  TensorPtr src = in;
  if (outer != 1) {
    // bring the scatter dim to the front in rank-block order: [n, outer, len/n, inner]
    int64_t lenPer = in->shape[d] / n, inner = static_cast<int64_t>(prod(in->shape, d + 1, rank));
    std::vector<uint32_t> shape = {n, static_cast<uint32_t>(outer), static_cast<uint32_t>(lenPer * inner)};
    std::vector<int64_t> strides = {lenPer * inner, static_cast<int64_t>(in->shape[d]) * inner, 1};
    src = stridedView(in, shape, strides, 0, in->dtype);
  }
  if (dev->locals.size() > 1) TTB_CALL(ttb_group_start());
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_reduce_scatter(r.comm, src->shards[i]->ptr, out->shards[i]->ptr, out->volume(), ttbDtype(in->dtype),
                                static_cast<int>(op->reduce_type()), r.stream));
  });
  if (dev->locals.size() > 1) TTB_CALL(ttb_group_end());
  put(op->out(), out);
}

// Replicated along the axis -> each coordinate keeps its 1/n slice of `dim` (tools/golden/mapping.py:5751-5794).
void Executor::runMeshPartition(const fbt::MeshPartitionOp *op) {
  TensorPtr in = getDevice(op->in());
  uint32_t axis = op->cluster_axis().value_or(dev->meshShape[0] > 1 ? 0 : 1);
  uint32_t n = meshAxisSize(axis);
  if (n == 1) {
    put(op->out(), in);
    return;
  }
  size_t rank = in->shape.size();
  int d = normDim(op->dim(), rank);
  TTRT_ASSERT(in->shape[d] % n == 0, "partition dimension must divide by the mesh axis size");
  std::vector<uint32_t> outShape = in->shape;
  outShape[d] /= n;
  std::vector<int64_t> dense = denseStrides(in->shape);
  TensorPtr out = makeDeviceTensor(dev, outShape, in->dtype);
  std::vector<int64_t> shape(outShape.begin(), outShape.end());
  eachRank([&](size_t i, const RankCtx &r) {
    int64_t offset = static_cast<int64_t>(r.meshRank) * outShape[d] * dense[d];
    TTB_CALL(ttb_strided_copy(in->shards[i]->ptr, out->shards[i]->ptr, static_cast<int>(dataTypeSize(in->dtype)),
                              static_cast<int>(rank), shape.data(), dense.data(), offset, r.stream));
  });
  put(op->out(), out);
}

// Host full tensor -> one shard per mesh coordinate (ttir.mesh_shard full_to_shard,
// lib/Conversion/TTIRToTTNN/TTIRToTTNN.cpp:2770-2817): placement i says what mesh axis i does.
void Executor::runDistribute(const fbt::DistributeTensorOp *op) {
  TensorPtr in = get(op->in());
  TTRT_ASSERT(op->mapper_config() && op->mapper_config()->placements(), "distribute_tensor without placements");
  const auto *pl = op->mapper_config()->placements();
  TTRT_ASSERT(pl->size() == 2, "placements must cover both mesh axes");
  // Only one mesh axis is larger than 1; find the tensor dim sharded over it (or none).
  int shardDim = -1;
  for (uint32_t ax = 0; ax < 2; ++ax) {
    fbt::Placement p = pl->Get(ax);
    if (p.type() == fbt::PlacementType::Shard && dev->meshShape[ax] > 1) shardDim = normDim(p.dim(), in->shape.size());
  }
  uint32_t n = dev->worldSize;
  std::vector<uint32_t> outShape = in->shape;
  if (shardDim >= 0) {
    TTRT_ASSERT(outShape[shardDim] % n == 0, "sharded dimension ", shardDim, " (", outShape[shardDim], ") must divide by ", n);
    outShape[shardDim] /= n;
  }
  TTRT_ASSERT(outShape == refShape(op->out()), "distribute_tensor result shape differs from the op's result type");
  bool toDev = refOnDevice(op->out());
  if (shardDim < 0) {
    // replicate
    TensorPtr out = in;
    if (toDev && in->storage == Storage::Host) out = toDevice(in, dev, in->dtype);
    put(op->out(), out);
    return;
  }
  TTRT_ASSERT(in->storage == Storage::Host, "input of distribute_tensor must be on host");
  TTRT_ASSERT(in->shards.size() == 1, "input of distribute_tensor is already distributed");
  // Slice on the host into per-coordinate shards; only the coordinates this process owns are built.
  size_t es = dataTypeSize(in->dtype);
  size_t outer = prod(in->shape, 0, shardDim), lenPer = outShape[shardDim], inner = prod(in->shape, shardDim + 1, in->shape.size());
  size_t rowBytes = lenPer * inner * es, fullRowBytes = static_cast<size_t>(in->shape[shardDim]) * inner * es;
  auto host = std::make_shared<TensorImpl>();
  host->shape = outShape;
  host->stride = denseStrides(outShape);
  host->dtype = in->dtype;
  host->storage = Storage::Host;
  host->shards.resize(n);
  const uint8_t *src = static_cast<const uint8_t *>(in->shards[0]->ptr);
  for (const RankCtx &r : dev->locals) {
    TensorPtr piece = makeHostTensor(outShape, in->dtype, 1);
    uint8_t *dst = static_cast<uint8_t *>(piece->shards[0]->ptr);
    for (size_t o = 0; o < outer; ++o) {
      std::memcpy(dst + o * rowBytes, src + o * fullRowBytes + r.meshRank * rowBytes, rowBytes);
    }
    host->shards[r.meshRank] = piece->shards[0];
  }
  if (toDev) {
    // toDevice indexes shards by mesh coordinate; absent coordinates belong to other processes.
    TensorPtr out = toDevice(host, dev, in->dtype);
    out->layout = refLayout(op->out());
    put(op->out(), out);
  } else {
    put(op->out(), host);
  }
}

// Shards -> full tensor on the host (ttir.mesh_shard shard_to_full, TTIRToTTNN.cpp:2819-2888):
// dims[i] is the tensor dim concatenated over mesh axis i; an override extent of 1 means
// "replicated on that axis, take the first".
void Executor::runAggregate(const fbt::AggregateTensorOp *op) {
  TensorPtr in = get(op->in());
  TTRT_ASSERT(op->composer_config() && op->composer_config()->dims(), "aggregate_tensor without composer dims");
  const auto *dims = op->composer_config()->dims();
  const auto *ovr = op->composer_config()->mesh_shape_override();
  int catDim = -1;
  for (uint32_t ax = 0; ax < dims->size() && ax < 2; ++ax) {
    uint32_t extent = (ovr && ax < ovr->size()) ? ovr->Get(ax) : dev->meshShape[ax];
    if (extent > 1) catDim = normDim(dims->Get(ax), in->shape.size());
  }
  uint32_t n = dev->worldSize;
  if (catDim < 0 || n == 1) {
    // replicated: any one shard is the result
    TensorPtr h = in->storage == Storage::Device ? toHostTensor(in, true) : in;
    auto one = std::make_shared<TensorImpl>();
    one->shape = h->shape;
    one->stride = h->stride;
    one->dtype = h->dtype;
    one->storage = Storage::Host;
    one->shards.push_back(h->shards[0]);
    put(op->out(), one);
    return;
  }
  std::vector<uint32_t> outShape = in->shape;
  outShape[catDim] *= n;
  TTRT_ASSERT(outShape == refShape(op->out()), "aggregate_tensor result shape differs from the op's result type");
  size_t es = dataTypeSize(in->dtype);
  size_t outer = prod(in->shape, 0, catDim), rowBytes = prod(in->shape, catDim, in->shape.size()) * es;
  TensorPtr out = makeHostTensor(outShape, in->dtype, 1);
  uint8_t *dst = static_cast<uint8_t *>(out->shards[0]->ptr);
  if (dev->multiProcess) {
    // Each process holds one shard: gather them on the device, then read back once.
    TensorPtr d = in->storage == Storage::Device ? in : toDevice(in, dev, in->dtype);
    TensorPtr all = makeDeviceTensor(dev, {n, static_cast<uint32_t>(in->volume())}, in->dtype);
    const RankCtx &r = dev->locals[0];
    TTB_CALL(ttb_set_device(r.cudaDevice));
    TTB_CALL(ttb_all_gather(r.comm, d->shards[0]->ptr, all->shards[0]->ptr, in->volume(), ttbDtype(in->dtype), r.stream));
    TensorPtr h = toHostTensor(all, true);
    const uint8_t *src = static_cast<const uint8_t *>(h->shards[0]->ptr);
    for (uint32_t k = 0; k < n; ++k)
      for (size_t o = 0; o < outer; ++o)
        std::memcpy(dst + (o * n + k) * rowBytes, src + (static_cast<size_t>(k) * outer + o) * rowBytes, rowBytes);
  } else {
    TensorPtr h = in->storage == Storage::Device ? toHostTensor(in, true) : in;
    TTRT_ASSERT(h->shards.size() == n, "aggregate_tensor needs one shard per mesh coordinate");
    for (uint32_t k = 0; k < n; ++k) {
      const uint8_t *src = static_cast<const uint8_t *>(h->shards[k]->ptr);
      for (size_t o = 0; o < outer; ++o) std::memcpy(dst + (o * n + k) * rowBytes, src + o * rowBytes, rowBytes);
    }
  }
  put(op->out(), out);
}

// ---- sub-programs: const-eval cache, calls, traces --------------------------------------------------
// A program of the same binary run on behalf of an op of this one (the reference constructs a
// nested ProgramExecutor the same way: operations/cache/load_cached.cpp:71-75,
// operations/mlir_native/func_call.cpp:25-31).
std::vector<TensorPtr> Executor::runSubProgram(uint32_t index, const std::vector<TensorPtr> &inputs) {
  std::vector<Tensor> in;
  in.reserve(inputs.size());
  for (const TensorPtr &t : inputs) in.push_back(wrapTensor(t));
  Executor sub(dev, bin, index, in);
  std::vector<Tensor> out = sub.run();
  std::vector<TensorPtr> res;
  res.reserve(out.size());
  for (const Tensor &t : out) res.push_back(unwrapTensor(t));
  return res;
}

// LoadCachedOp (operations/cache/load_cached.cpp:20-91): the outputs of a const-eval program are
// computed once per (device, program hash, versions of the inputs) and kept, retained, in a
// process-wide cache; later submits of any binary with the same function bind the cached tensors.
void Executor::runLoadCached(const fbt::LoadCachedOp *op) {
  ConstEvalKey key;
  key.device = dev.get();
  key.hash = op->program_hash() ? op->program_hash()->str() : std::string();
  if (key.hash.empty()) {
    // no hash in the file: the function is only shared within this binary
    key.hash = strcat_("binary", bin.id(), ":", op->callee_name() ? op->callee_name()->str() : "", ":", op->program_idx());
  }
  std::vector<TensorPtr> ins, roots;
  if (op->inputs()) {
    for (const auto *ref : *op->inputs()) {
      TensorPtr t = get(ref);
      TensorPtr root = t->base ? t->base : t;
      key.inputVersions.push_back(root->version.load());
      ins.push_back(t);
      roots.push_back(root);
    }
  }
  std::vector<TensorPtr> outs;
  if (!ConstEvalCache::get().find(key, outs)) {
    refuseWhileRecording("evaluating a const-eval function");
    outs = runSubProgram(op->program_idx(), ins);
    for (const TensorPtr &t : outs) t->retain = true; // DeallocateOps of any program leave them alone
    ConstEvalCache::get().store(key, roots, outs);
  }
  uint32_t nOut = op->outputs() ? op->outputs()->size() : 0;
  TTRT_ASSERT(outs.size() == nOut, "const-eval function returned ", outs.size(), " tensors, the op declares ", nOut);
  for (uint32_t i = 0; i < nOut; ++i) put(op->outputs()->Get(i), outs[i]);
}

void Executor::runFuncCall(const fbt::FuncCallOp *op) {
  TTRT_ASSERT(!op->semaphore_inputs() || op->semaphore_inputs()->size() == 0,
              "global semaphores are a Tenstorrent fabric object and have no counterpart here");
  std::vector<TensorPtr> ins;
  if (op->inputs()) {
    for (const auto *ref : *op->inputs()) ins.push_back(get(ref));
  }
  std::vector<TensorPtr> outs = runSubProgram(op->program_id(), ins);
  uint32_t nOut = op->outputs() ? op->outputs()->size() : 0;
  TTRT_ASSERT(outs.size() == nOut, "Number of outputs does not match");
  for (uint32_t i = 0; i < nOut; ++i) put(op->outputs()->Get(i), outs[i]);
}

void Executor::refuseWhileRecording(const char *what) const {
  TTRT_ASSERT(dev->recordingTrace == 0, what, " is not possible while a trace is being recorded");
}

static TensorPtr traceIdTensor(uint32_t id) {
  TensorPtr t = makeHostTensor({}, DataType::UInt32, 1);
  *static_cast<uint32_t *>(t->shards[0]->ptr) = id;
  return t;
}

static uint32_t traceIdOf(const TensorPtr &t) {
  TTRT_ASSERT(t && t->storage == Storage::Host && t->dtype == DataType::UInt32 && t->volume() == 1 && t->allocated(),
              "Trace ID must be UINT32");
  return *static_cast<const uint32_t *>(t->shards[0]->ptr);
}

// BeginTraceCaptureOp (operations/trace/begin_trace_capture.cpp:12-27): from here to the matching
// EndTraceCaptureOp the compute stream records instead of running.  The trace id is a host scalar.
void Executor::runBeginTraceCapture(const fbt::BeginTraceCaptureOp *op) {
  TTRT_ASSERT(dev->recordingTrace == 0, "a trace is already being recorded on this device");
  TTRT_ASSERT(!dev->multiProcess, "traces are recorded by the process that owns the whole mesh");
  uint32_t id = dev->nextTraceId++;
  size_t begun = 0;
  try {
    eachRank([&](size_t, const RankCtx &r) {
      TTB_CALL(ttb_trace_begin(r.stream));
      ++begun;
    });
  } catch (...) {
    for (size_t i = 0; i < begun; ++i) ttb_trace_abort(dev->locals[i].stream);
    throw;
  }
  dev->recordingTrace = id;
  put(op->trace_id(), traceIdTensor(id));
}

void Executor::runEndTraceCapture(const fbt::EndTraceCaptureOp *op) {
  uint32_t id = traceIdOf(get(op->trace_id()));
  TTRT_ASSERT(id != 0 && id == dev->recordingTrace, "EndTraceCaptureOp names trace ", id, " but trace ",
              dev->recordingTrace, " is being recorded");
  dev->recordingTrace = 0;
  TraceGraph g;
  g.execs.assign(dev->locals.size(), nullptr);
  std::string failure;
  for (size_t i = 0; i < dev->locals.size(); ++i) {
    ttb_set_device(dev->locals[i].cudaDevice);
    if (!failure.empty()) {
      ttb_trace_abort(dev->locals[i].stream);
    } else if (ttb_trace_end(dev->locals[i].stream, &g.execs[i]) != TTB_OK) {
      failure = ttb_last_error();
    }
  }
  if (!failure.empty()) {
    for (void *e : g.execs) ttb_trace_destroy(e);
    TTRT_FATAL("recording trace ", id, " failed: ", failure);
  }
  dev->traces[id] = std::move(g);
}

void Executor::runExecuteTrace(const fbt::ExecuteTraceOp *op) {
  uint32_t id = traceIdOf(get(op->trace_id()));
  refuseWhileRecording("replaying a trace");
  auto it = dev->traces.find(id);
  TTRT_ASSERT(it != dev->traces.end(), "no recorded trace has id ", id);
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_trace_launch(it->second.execs.at(i), r.stream));
    if (op->blocking()) TTB_CALL(ttb_stream_sync(r.stream));
  });
}

// Brings the trace's persistent input slots up to date with the op's current inputs
// (operations/trace/capture_or_execute_trace.cpp:98-154): a slot whose version equals its input's
// is left alone; otherwise the input is copied in (device to device for constants, parameters and
// caches the caller replaced; host to device for everything else) and the versions are synchronised.
void Executor::updateTraceInputSlots(const fbt::CaptureOrExecuteTraceOp *op, std::vector<TensorPtr> &slots,
                                     bool residentOnly) {
  uint32_t nIn = op->inputs() ? op->inputs()->size() : 0;
  TTRT_ASSERT(slots.size() == nIn, "Mismatched number of inputs, expected: ", nIn, " got: ", slots.size());
  for (uint32_t i = 0; i < nIn; ++i) {
    const auto *ref = op->inputs()->Get(i);
    bool resident = refOnDevice(ref);
    if (residentOnly && !resident) continue;
    TensorPtr in = get(ref);
    TensorPtr root = in->base ? in->base : in;
    TensorPtr &slot = slots[i];
    if (root->version.load() == slot->version.load()) continue;
    TTRT_ASSERT(in->volume() == slot->volume() && in->dtype == slot->dtype, "trace input ", i,
                " does not match its slot in size or data type");
    if (resident) {
      TTRT_ASSERT(in->storage == Storage::Device, "trace input ", i, " is declared device-resident but lives on the host");
      orderAfterUploads(in);
      eachRank([&](size_t r_, const RankCtx &r) {
        if (in->shards[r_]->ptr != slot->shards[r_]->ptr) {
          TTB_CALL(ttb_memcpy_d2d(slot->shards[r_]->ptr, in->shards[r_]->ptr, slot->bytes(), r.stream));
        }
      });
    } else {
      TensorPtr h = in->storage == Storage::Device ? toHostTensor(in, true) : in;
      eachRank([&](size_t r_, const RankCtx &r) {
        const BufferPtr &src = h->shards.size() == 1 ? h->shards[0] : h->shards.at(r.meshRank);
        TTB_CALL(ttb_memcpy_h2d(slot->shards[r_]->ptr, src->ptr, slot->bytes(), r.stream));
      });
    }
    slot->version.store(root->version.load());
  }
}

// CaptureOrExecuteTraceOp (operations/trace/capture_or_execute_trace.cpp:264-355).  First visit:
// the slot-allocation program creates the persistent input and output buffers, the capture
// program fills the host-staged slots, runs the traced function once normally and once recording,
// and replays the recording; later visits refresh the input slots and replay.  The recorded graph
// owns the memory of its intermediates, so allocations made elsewhere between two replays cannot
// invalidate it and a trace is never recorded twice (the reference re-records a trace whenever
// another one was recorded after it, because its traces bake in addresses of a shared allocator).
void Executor::runCaptureOrExecuteTrace(const fbt::CaptureOrExecuteTraceOp *op) {
  refuseWhileRecording("CaptureOrExecuteTraceOp");
  TTRT_ASSERT(!op->semaphore_inputs() || op->semaphore_inputs()->size() == 0,
              "global semaphores are a Tenstorrent fabric object and have no counterpart here");
  uint32_t nIn = op->inputs() ? op->inputs()->size() : 0;
  uint32_t nOut = op->outputs() ? op->outputs()->size() : 0;
  TraceKey key{bin.id(), programIndex, op->capture_program_id(), op->execute_program_id()};
  auto publish = [&](const TraceData &td) {
    TTRT_ASSERT(td.outputSlots.size() == nOut, "Mismatched number of outputs, expected: ", nOut, " got: ",
                td.outputSlots.size());
    for (uint32_t i = 0; i < nOut; ++i) put(op->outputs()->Get(i), td.outputSlots[i]);
  };
  auto it = dev->traceCache.find(key);
  if (it == dev->traceCache.end()) {
    debug::Stats::get().incrementStat("TraceCacheMiss");
    std::vector<TensorPtr> resident, staged;
    for (uint32_t i = 0; i < nIn; ++i) {
      const auto *ref = op->inputs()->Get(i);
      (refOnDevice(ref) ? resident : staged).push_back(get(ref));
    }
    std::vector<TensorPtr> slots = runSubProgram(op->allocate_slots_program_id(), resident);
    TTRT_ASSERT(slots.size() == size_t(nIn) + nOut, "Mismatched number of trace slots, expected: ", nIn + nOut,
                " got: ", slots.size());
    for (const TensorPtr &t : slots) t->retain = true; // owned by the trace cache from here on
    TraceData td;
    td.inputSlots.assign(slots.begin(), slots.begin() + nIn);
    td.outputSlots.assign(slots.begin() + nIn, slots.end());
    updateTraceInputSlots(op, td.inputSlots, /*residentOnly=*/true);
    // capture program arguments: host-staged inputs, input slots, output slots
    std::vector<TensorPtr> args = staged;
    args.insert(args.end(), td.inputSlots.begin(), td.inputSlots.end());
    args.insert(args.end(), td.outputSlots.begin(), td.outputSlots.end());
    std::vector<TensorPtr> res = runSubProgram(op->capture_program_id(), args);
    TTRT_ASSERT(res.size() == 1, "Capture program must return exactly the new trace id, got: ", res.size());
    td.traceId = traceIdOf(res[0]);
    TTRT_ASSERT(dev->traces.count(td.traceId), "the capture program returned an id that names no recorded trace");
    publish(td); // the capture program replays once, so the output slots hold this call's results
    dev->traceCache.emplace(key, std::move(td));
    debug::Stats::get().incrementStat("CapturedTrace");
    return;
  }
  TraceData &td = it->second;
  updateTraceInputSlots(op, td.inputSlots, /*residentOnly=*/false);
  std::vector<TensorPtr> res = runSubProgram(op->execute_program_id(), {traceIdTensor(td.traceId)});
  (void)res;
  publish(td);
  debug::Stats::get().incrementStat("ExecutedTrace");
}

// WriteTensorOp: the contents of a host tensor go into an existing device tensor (the capture
// program fills the host-staged trace slots with it before recording starts).
void Executor::runWriteTensor(const fbt::WriteTensorOp *op) {
  refuseWhileRecording("a host-to-device write");
  TensorPtr h = get(op->host_tensor());
  TensorPtr d = get(op->device_tensor());
  if (h->storage == Storage::Device) h = toHostTensor(h, true);
  TTRT_ASSERT(d->storage == Storage::Device && d->allocated(), "write_tensor needs an allocated device tensor");
  TTRT_ASSERT(h->volume() == d->volume() && h->dtype == d->dtype, "write_tensor needs equal size and data type");
  orderAfterUploads(d);
  eachRank([&](size_t r_, const RankCtx &r) {
    const BufferPtr &src = h->shards.size() == 1 ? h->shards[0] : h->shards.at(r.meshRank);
    TTB_CALL(ttb_memcpy_h2d(d->shards[r_]->ptr, src->ptr, d->bytes(), r.stream));
    if (op->blocking()) TTB_CALL(ttb_stream_sync(r.stream));
  });
  TensorPtr root = d->base ? d->base : d;
  root->version.store(TensorImpl::nextTensorVersion());
}

// CopyOp: device-to-device copy into an existing tensor (the traced function stores its results
// into the persistent output slots with it).
void Executor::runCopy(const fbt::CopyOp *op) {
  TensorPtr src = getDevice(op->src());
  TensorPtr dst = get(op->dst());
  TTRT_ASSERT(dst->storage == Storage::Device && dst->allocated(), "copy needs an allocated device destination");
  TTRT_ASSERT(src->volume() == dst->volume() && src->dtype == dst->dtype, "copy needs equal size and data type");
  bool same = true;
  for (size_t i = 0; i < dev->locals.size(); ++i) same = same && src->shards[i]->ptr == dst->shards[i]->ptr;
  if (same) return; // the producer already wrote into the destination
  eachRank([&](size_t i, const RankCtx &r) {
    TTB_CALL(ttb_memcpy_d2d(dst->shards[i]->ptr, src->shards[i]->ptr, dst->bytes(), r.stream));
  });
}

std::vector<Tensor> runProgram(const std::shared_ptr<DeviceImpl> &dev, Binary &binary, uint32_t programIndex,
                               std::vector<Tensor> &inputs) {
  std::lock_guard<std::mutex> g(dev->submitMutex);
  try {
    Executor ex(dev, binary, programIndex, inputs);
    return ex.run();
  } catch (...) {
    // A failure between BeginTraceCaptureOp and EndTraceCaptureOp leaves the streams recording.
    if (dev->recordingTrace != 0) {
      for (const RankCtx &r : dev->locals) {
        ttb_set_device(r.cudaDevice);
        ttb_trace_abort(r.stream);
      }
      dev->recordingTrace = 0;
    }
    throw;
  }
}

} // namespace tt::runtime::cuda

// ---- hook-facing API (runtime.h:246-283 of the reference) --------------------------------------------------------
namespace tt::runtime {

using namespace ::tt::runtime::cuda;
namespace fbt = ::tt::target::ttnn;

static const fbt::Operation *opOf(const OpContext &c) { return c.as<OpContextImpl>(DeviceRuntime::CUDA).op; }
static Executor *execOf(const CallbackContext &c) { return c.as<ProgramContextImpl>(DeviceRuntime::CUDA).executor; }

static TensorRef wrapRef(const fbt::TensorRef *r) {
  return TensorRef(std::shared_ptr<void>(const_cast<fbt::TensorRef *>(r), [](void *) {}), DeviceRuntime::CUDA);
}
static const fbt::TensorRef *unwrapRef(const TensorRef &r) { return &r.as<fbt::TensorRef>(DeviceRuntime::CUDA); }

std::string getOpDebugString(OpContext c) {
  const auto *op = opOf(c);
  return op->debug_info() ? op->debug_info()->str() : "";
}

std::string getOpLocInfo(OpContext c) {
  const auto *op = opOf(c);
  return op->loc_info() ? op->loc_info()->str() : "";
}

std::vector<TensorRef> getOpOutputRefs(OpContext c) {
  std::vector<const fbt::TensorRef *> ins, outs;
  collectOpRefs(opOf(c), ins, outs);
  if (opOf(c)->type_type() == fbt::OpType::DeallocateOp) outs.clear();
  std::vector<TensorRef> r;
  for (const auto *o : outs) r.push_back(wrapRef(o));
  return r;
}

std::vector<TensorRef> getOpInputRefs(OpContext c) {
  std::vector<const fbt::TensorRef *> ins, outs;
  collectOpRefs(opOf(c), ins, outs);
  std::vector<TensorRef> r;
  for (const auto *i : ins) r.push_back(wrapRef(i));
  return r;
}

std::vector<uint32_t> getTensorRefShape(TensorRef ref) {
  std::vector<uint32_t> s;
  const auto *r = unwrapRef(ref);
  if (r->desc() && r->desc()->shape()) {
    for (int32_t d : *r->desc()->shape()) s.push_back(static_cast<uint32_t>(d));
  }
  return s;
}

::tt::target::DataType getTensorRefDataType(TensorRef ref) {
  return unwrapRef(ref)->desc()->layout()->memory_desc()->data_type();
}

std::optional<Tensor> retrieveTensorFromPool(CallbackContext ctx, TensorRef ref, bool) {
  Executor *ex = execOf(ctx);
  auto it = ex->pool.find(unwrapRef(ref)->global_id());
  if (it == ex->pool.end() || !it->second->allocated()) {
    return std::nullopt;
  }
  TensorPtr t = it->second;
  if (t->storage == Storage::Device) {
    TensorPtr h = toHostTensor(t, true);
    auto one = std::make_shared<TensorImpl>();
    one->shape = h->shape;
    one->stride = h->stride;
    one->dtype = h->dtype;
    one->storage = Storage::Host;
    one->shards.push_back(h->shards[0]);
    return wrapTensor(one);
  }
  return wrapTensor(t);
}

std::unordered_map<std::uint32_t, Tensor> getOpOutputTensor(OpContext c, CallbackContext ctx) {
  std::unordered_map<std::uint32_t, Tensor> out;
  Executor *ex = execOf(ctx);
  std::vector<const fbt::TensorRef *> ins, outs;
  collectOpRefs(opOf(c), ins, outs);
  if (outs.empty() || opOf(c)->type_type() == fbt::OpType::DeallocateOp) {
    return out;
  }
  auto it = ex->pool.find(outs[0]->global_id());
  if (it == ex->pool.end() || !it->second->allocated()) {
    return out;
  }
  TensorPtr t = it->second;
  TensorPtr h = t->storage == Storage::Device ? toHostTensor(t, true) : t;
  for (size_t i = 0; i < h->shards.size(); ++i) {
    auto one = std::make_shared<TensorImpl>();
    one->shape = h->shape;
    one->stride = h->stride;
    one->dtype = h->dtype;
    one->storage = Storage::Host;
    one->shards.push_back(h->shards[i]);
    uint32_t coord = t->storage == Storage::Device ? ex->dev->locals[i].meshRank : static_cast<uint32_t>(i);
    out.emplace(coord, wrapTensor(one));
  }
  return out;
}

void updateTensorInPool(CallbackContext ctx, TensorRef ref, Tensor srcTensor) {
  Executor *ex = execOf(ctx);
  auto it = ex->pool.find(unwrapRef(ref)->global_id());
  TTRT_ASSERT(it != ex->pool.end(), "tensor ", unwrapRef(ref)->global_id(), " is not in the pool");
  TensorPtr dst = it->second;
  TensorPtr src = unwrapTensor(srcTensor);
  TTRT_ASSERT(src->volume() == dst->volume(), "replacement tensor has a different element count");
  Tensor d = wrapTensor(dst);
  if (src->dtype != dst->dtype) {
    // normalise on the host
    std::vector<uint8_t> tmp(dst->bytes());
    memcpy(tmp.data(), srcTensor, dst->dtype);
    Tensor h = createOwnedHostTensor(tmp.data(), dst->shape, dst->stride, dataTypeSize(dst->dtype), dst->dtype);
    auto hi = unwrapTensor(h);
    if (dst->shards.size() > 1) {
      for (size_t i = 1; i < dst->shards.size(); ++i) hi->shards.push_back(hi->shards[0]);
    }
    memcpy(d, h);
  } else {
    if (src->shards.size() == 1 && dst->shards.size() > 1) {
      auto rep = std::make_shared<TensorImpl>();
      rep->shape = src->shape;
      rep->stride = src->stride;
      rep->dtype = src->dtype;
      rep->storage = src->storage;
      rep->device = src->device;
      for (size_t i = 0; i < dst->shards.size(); ++i) rep->shards.push_back(src->shards[0]);
      memcpy(d, wrapTensor(rep));
    } else {
      memcpy(d, srcTensor);
    }
  }
}

size_t getProgramIndex(CallbackContext ctx) { return execOf(ctx)->programIndex; }

void walkProgram(Binary bin, uint32_t programIndex, const OpWalkFn &cb) {
  const auto *programs = bin.get()->programs();
  TTRT_ASSERT(programs && programIndex < programs->size(), "program index out of range");
  const auto *ops = programs->Get(programIndex)->operations();
  if (!ops) return;
  for (const auto *op : *ops) {
    auto impl = std::make_shared<OpContextImpl>();
    impl->op = op;
    cb(OpContext(std::static_pointer_cast<void>(impl), DeviceRuntime::CUDA));
  }
}

} // namespace tt::runtime
