// The dlx model format: in-memory messages and a proto3 wire reader/writer.
//
// A dlx file is the binary protobuf encoding of dlxnet.ModelProto
// (ogl_runtime/opengl/core/dlxnet.proto:1-215; the converter's
// converter/core/dlcl.proto is the same schema). The reference reads it with
// generated protobuf code (ogl_runtime/opengl/utils/protobuf.cc:10-27); this
// runtime has no protobuf dependency and decodes the wire format directly, so a
// file written by the existing converter loads unchanged. Field numbers below
// are the schema's.
#ifndef OGLE_RUNTIME_DLX_H_
#define OGLE_RUNTIME_DLX_H_
#include <cstdint>
#include <string>
#include <vector>

namespace dlxnet {

struct TensorProto {
    enum DataFormat { NCHW = 0, NHWC = 1, NHWC4 = 3, HWN4C4 = 4, ANY = 5, ANY4 = 6 };
    enum DataType { FLOAT32 = 0, FLOAT16 = 1, INT32 = 2, INT8 = 3 };
    DataFormat data_format = NCHW;          // field 1
    DataType data_type = FLOAT32;           // field 2
    std::vector<int32_t> dims;              // field 3
    std::vector<float> float_data;          // field 4 (packed)
    std::vector<int32_t> int32_data;        // field 5 (packed)
    std::vector<int64_t> int64_data;        // field 7 (packed)
    DataFormat target_data_format = NCHW;   // field 8
};

struct Conv2dAttribute {
    std::vector<int64_t> kernel_shape, strides, pads, dilations;  // 1..4
    int64_t group = 0;                                             // 5
    std::string activation_type;                                   // 6
    float min = 0.f, max = 0.f;                                    // 7, 8
};
struct ConstAttribute { TensorProto value; };                      // 1
struct BatchNormAttribute { float momentum = 0.f, epsilon = 0.f; };  // 1, 2
struct ReluAttribute { float slope = 0.f; };
struct MaxPoolAttribute { std::vector<int64_t> kernel_shape, strides, pads; };  // 1..3
struct AvePoolAttribute { std::vector<int64_t> kernel_shape, strides, pads; };
struct BinaryAttribute { std::string binary_op_type; };
struct FlattenAttribute { int32_t axis = 0; };
struct ClipAttribute { float min = 0.f, max = 0.f; };
struct TransposeAttribute { std::vector<int32_t> perm; };
struct GemmAttribute { float alpha = 0.f, beta = 0.f; int32_t transb = 0; };
struct InputAttribute { std::vector<int32_t> dims; };              // field 3
struct UnsqueezeAttribute { std::vector<int32_t> axes; };
struct ConcatAttribute { int32_t axis = 0; };
struct ReshapeAttribute { int32_t axis = 0; };
struct GatherAttribute { int32_t axis = 0; };

// All sub-messages are optional in the schema; absent ones keep their defaults,
// which is also what the generated accessors return.
struct Attribute {
    Conv2dAttribute conv2d_attr;        // 1
    ConstAttribute const_attr;          // 2
    BatchNormAttribute batchnorm_attr;  // 3
    ReluAttribute relu_attr;            // 4
    MaxPoolAttribute maxpool_attr;      // 5
    AvePoolAttribute avepool_attr;      // 6
    FlattenAttribute flatten_attr;      // 7
    BinaryAttribute binary_attr;        // 8
    GemmAttribute gemm_attr;            // 9
    InputAttribute input_attr;          // 10
    ClipAttribute clip_attr;            // 11
    TransposeAttribute transpose_attr;  // 12
    // 13 shape_attr (empty message)
    GatherAttribute gather_attr;        // 14
    UnsqueezeAttribute unsqueeze_attr;  // 15
    ConcatAttribute concat_attr;        // 16
    ReshapeAttribute reshape_attr;      // 17
};

struct NodeProto {
    std::vector<int64_t> input_index;   // 1
    std::vector<int64_t> output_index;  // 2
    Attribute attr;                     // 3
    std::string doc_string;             // 4
    std::string name;                   // 5
    std::string type;                   // 6
};

struct GraphProto {
    std::vector<NodeProto> node;            // 1
    std::string name;                       // 2
    std::vector<std::string> tensor_names;  // 3
    std::vector<std::string> output_names;  // 4
    std::vector<std::string> input_names;   // 5
};

struct ModelProto {
    GraphProto graph;            // 1
    std::string version;         // 2
    std::string producer_name;   // 3
    std::string doc_string;      // 4
};

// Decodes a serialized ModelProto. Unknown fields are skipped, as protobuf does.
// Returns false and fills *error on malformed input.
bool ParseModel(const void* data, size_t size, ModelProto* model, std::string* error);
bool ReadModelFromFile(const std::string& path, ModelProto* model, std::string* error);
// Encodes in field-number order with packed repeated scalars (what protoc-generated
// proto3 code emits).
std::string SerializeModel(const ModelProto& model);

}  // namespace dlxnet
#endif
