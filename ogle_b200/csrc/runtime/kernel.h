// Kernel: the per-operator interface, as ogl_runtime/opengl/core/kernel.h:15-123.
// A subclass parses its attributes (SetupAttr), picks a variant and output data
// formats once input tensors are known (SelectKernel), infers output shapes
// (InferOutputShape) and enqueues its work (Compute). Compute calls one entry
// point of include/ogle_cuda.h on the session's stream; it never allocates or
// synchronises, so the session can capture the whole sequence in a CUDA graph.
#ifndef OGLE_RUNTIME_KERNEL_H_
#define OGLE_RUNTIME_KERNEL_H_
#include "context.h"
#include "types.h"

namespace ogle {

class FBOSession;

class Kernel {
public:
    explicit Kernel(Context* context) : context_(context) {}
    virtual ~Kernel() {}

    virtual void Compute(TensorList& inputs, TensorList& outputs) = 0;
    virtual void SetupAttr(const dlxnet::Attribute& attr) = 0;
    virtual void Setup(const dlxnet::NodeProto& node_proto, FBOSession* session);
    void Compute() { Compute(input_tensors_, output_tensors_); }

    DataFormat GetOutputDFormat(int i) const;
    std::string DebugString() const;

    virtual void InferOutputShape(TensorShapeList& inputs, TensorShapeList& outputs) = 0;
    // some ops need input values or data formats (Reshape, Pool, Concat)
    virtual void InferOutputShape(const TensorList& inputs, TensorShapeList& output_shapes);

    void set_kernel_name(const std::string& n) { kernel_name_ = n; }
    void set_kernel_type(const std::string& n) { kernel_type_ = n; }
    const std::string& kernel_name() const { return kernel_name_; }
    const std::string& kernel_type() const { return kernel_type_; }
    void set_session(FBOSession* s) { session_ = s; }
    FBOSession* session() const { return session_; }

    // Shape-like kernels run at setup whatever their inputs' state (kernel.h:80).
    virtual bool ForceReady() const { return false; }
    // Name of the device kernel family chosen by SelectKernel (the reference
    // stores a shader file name here).
    const std::string& kernel_fname() const { return kernel_fname_; }
    virtual void SelectKernel(const TensorList& inputs) {}
    // True when Compute only aliases/keeps memory and launches nothing.
    virtual bool IsNoOp() const { return false; }
    // Offered a later node of the steady-state sequence: return true to take over its work
    // (this kernel's Compute then also writes that node's outputs, and the session drops
    // the later node from the sequence).
    virtual bool AbsorbSibling(Kernel* later) { return false; }
    // Offered the only consumer of this kernel's output: return true to apply that node's
    // work in the same pass (this kernel's Compute then writes the consumer's output instead
    // of its own, which is no longer produced; the session drops the consumer).
    virtual bool AbsorbConsumer(Kernel* consumer) { return false; }
    // Residual blocks. An elementwise Add (with the activation it may have absorbed) describes itself:
    // the activation it applies and the tensor its result goes to.
    virtual bool AsResidualAdd(int* act, float* lo, float* hi, Tensor** dst) const { return false; }
    // Offered such an Add as the only reader of this kernel's output, and the Add's other operand (complete
    // before this kernel runs): return true to add that operand and apply the activation in this kernel's own
    // pass, writing `dst` (the session then drops the Add; this kernel's own tensor is no longer produced).
    virtual bool AbsorbResidualAdd(Kernel* add, Tensor* residual, Tensor* dst, int act, float lo, float hi) { return false; }
    // For AbsorbConsumer implementations: the activation a node applies, if it is one.
    virtual bool AsActivation(int* act, float* lo, float* hi) const { return false; }
    // Called once by the session after every tensor exists and the fusions are decided: a node may time
    // variants of its launch that give identical results (on its real tensors, whatever they hold) and keep
    // the fastest. Default: nothing to choose.
    virtual void Tune() {}
    // Concat in place. A concat-like node describes where its input i lies inside its output:
    // the input is `outer` rows of `chunk` floats, and row r belongs at
    // output + r * row_stride + offset (floats, padded layouts on both sides). False when the
    // node is no concat or the slice cannot be described that way.
    virtual bool ConcatPlacement(int input, long* outer, long* chunk, long* row_stride, long* offset) const { return false; }
    // Told that input i is written in place by its producer: Compute leaves that slice alone.
    virtual void InputPlaced(int input) {}
    // Offered to the producer of a tensor whose only reader is a concat: write the result into
    // `dst` with the geometry above instead of into this node's own output tensor (which is
    // then never written). Return true to accept.
    virtual bool PlaceOutput(Tensor* dst, long outer, long chunk, long row_stride, long offset) { return false; }

protected:
    // another node's output tensors, for AbsorbSibling / AbsorbConsumer implementations
    static const std::vector<Tensor*>& ConsumerOutputs(const Kernel* k) { return k->output_tensors_; }
    Context* context_;
    std::string kernel_fname_;
    std::vector<Tensor*> input_tensors_;    // not owned
    std::vector<Tensor*> output_tensors_;   // not owned
    std::vector<int> input_tensor_indexes_;
    std::vector<int> output_tensor_indexes_;
    std::vector<DataFormat> output_tensor_dformats_;
    std::vector<Kernel*> absorbed_;         // later nodes whose work this kernel took over (AbsorbSibling)
    std::vector<Tensor*> extra_writes_;     // tensors of other nodes this kernel writes into (PlaceOutput); not owned
    friend class FBOSession;
    std::string kernel_name_;
    std::string kernel_type_;
    FBOSession* session_ = nullptr;
};

}  // namespace ogle
#endif
