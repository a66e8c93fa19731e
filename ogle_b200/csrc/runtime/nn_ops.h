// Node-adding helpers over Scope with the names and argument meaning of the
// reference's ogl_runtime/opengl/nn/apis/nn_ops.h:10-68: every Add*Node appends one
// node named `name`, registers a tensor of the same name as its only output and
// returns that tensor's id; `input_ids` are tensor ids from earlier calls.
// The last block (pooling, batch norm, relu, add, decoder) has no counterpart in the
// reference's helper file; the operators themselves are the reference's.
#ifndef OGLE_RUNTIME_NN_OPS_H_
#define OGLE_RUNTIME_NN_OPS_H_
#include <string>
#include <vector>

#include "scope.h"
#include "tensor.h"

namespace ogle {

struct Conv2dParams {
    int kernel_size;
    int stride;
    int padding;
    int dilation;
    int groups;
    // fused activation as the converter's remapper writes it ("", "Relu" or "Clip")
    std::string activation_type;
    float min = 0.f, max = 0.f;
};
struct ConcatParams { int axis; };
struct TransposeParams { IntList perm; };
struct ClipParams { float min; float max; };
struct FlattenParams { int axis; };
struct GemmParams { float alpha; float beta; int transb; };
struct PoolParams { int kernel_size; int stride; int padding; };

int AddConstNode(Scope* scope, const std::string& name, const Tensor* cpu_tensor);
// Uniform [0,1) values from random(), as the reference's tests draw them.
int AddConstNode(Scope* scope, const std::string& name, const std::vector<int>& shape, DataFormat dst_dformat,
                 DataFormat src_dformat);
int AddConvNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const Conv2dParams& conv2d_params);
int AddInputNode(Scope* scope, std::string name);
int AddShapeNode(Scope* scope, std::string name, std::vector<int> input_ids);
int AddConcatNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const ConcatParams& concat_params);
int AddReshapeNode(Scope* scope, const std::string& name, std::vector<int> input_ids);
int AddTransposeNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const TransposeParams& trans_params);
int AddClipNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const ClipParams& clip_params);
int AddFlattenNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const FlattenParams& flatten_params);
int AddGemmNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const GemmParams& gemm_params);

int AddMaxPoolNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const PoolParams& pool_params);
int AddGlobalAveragePoolNode(Scope* scope, const std::string& name, std::vector<int> input_ids);
int AddBatchNormNode(Scope* scope, const std::string& name, std::vector<int> input_ids, float epsilon);
int AddReluNode(Scope* scope, const std::string& name, std::vector<int> input_ids);
int AddAddNode(Scope* scope, const std::string& name, std::vector<int> input_ids);
int AddDecoderNode(Scope* scope, const std::string& name, std::vector<int> input_ids);

}  // namespace ogle
#endif
