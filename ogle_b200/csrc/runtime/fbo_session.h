// FBOSession: loads a dlx graph, instantiates one Kernel per node through the
// registry, allocates every tensor once, pre-computes constant sub-graphs, and
// runs the remaining nodes in file order. Same public surface as the reference's
// ogl_runtime/opengl/core/fbo_session.h:11-90. The OpenGL framebuffer loop of
// fbo_session.cc:127-156 is replaced by a CUDA graph: the first Run executes the
// nodes eagerly, the next one captures them, later ones replay the capture.
#ifndef OGLE_RUNTIME_FBO_SESSION_H_
#define OGLE_RUNTIME_FBO_SESSION_H_
#include "context.h"
#include "kernel.h"
#include "types.h"

struct CUgraphExec_st;

namespace ogle {

struct NodeTiming {
    std::string name, type, kernel;
    float ms;
};

class FBOSession {
public:
    explicit FBOSession(Context* context);
    FBOSession() : FBOSession(GetContext()) {}
    virtual ~FBOSession();

    // Allocates tensors on the first call (shapes follow from the inputs given
    // then); uploads the inputs on every call.
    void Setup(const NamedTensorList& inputs_cpu);
    // Upload inputs, then run every node that is not pre-computed. Asynchronous:
    // returns when the work is enqueued on context()->stream().
    void Run(const NamedTensorList& inputs_cpu);
    // Run, but with inputs that already live on the device in NHWC4/ANY4 layout
    // (device-to-device copy into the session's input tensors).
    void RunDevice(const std::vector<std::pair<std::string, const float*>>& inputs_device);

    void LoadGraph(const dlxnet::ModelProto& model_proto);
    void LoadGraph(const std::string& model_path);

    // Reads named tensors back in the requested host formats ("NHWC", "NCHW",
    // "ANY", "NHWC4", "ANY4", "HWN4C4"). Allocates (*outputs)[i] when null; the
    // caller owns them. Synchronises.
    void GetOutputs(const TensorNameList& output_names, const StringList& output_dformats, TensorList* outputs);

    std::string DebugString() const;
    Context* context() const { return context_; }
    bool IsONNX() const { return model_.producer_name == "ONNX"; }
    Tensor* FindTensorByName(const std::string& name);
    Tensor* FindTensorById(int id);
    // true once the tensor was produced by the setup pass (a model constant or derived from one)
    bool IsTensorReady(int id) const { return id >= 0 && id < int(ready_.size()) && ready_[id]; }
    bool allow_resized() const { return allow_resized_; }
    void set_allow_resized(bool flag) { allow_resized_ = flag; }
    const IntList& default_input_sizes() const { return default_input_sizes_; }

    // CUDA-graph replay of the steady state (default on; OGLE_USE_GRAPH=0 disables).
    void set_use_graph(bool flag);
    bool graph_captured() const { return graph_exec_ != nullptr; }
    // Sibling fusion: nodes that read the same input with the same window (the SSD box and
    // class heads) run as one pass (default on; OGLE_FUSE_SIBLINGS=0 disables). Set before
    // the first Run.
    void set_fuse_siblings(bool flag) { fuse_siblings_ = flag; }
    int num_fused() const { return num_fused_; }
    // Activation fusion: a Relu or Clip that is the only reader of an Add's result is applied
    // in the Add's pass (a residual block's tail). The Add's own output tensor is then not
    // produced; GetOutputs on it fails with a message naming this switch (default on;
    // OGLE_FUSE_ACTIVATIONS=0 disables). Set before the first Run.
    void set_fuse_activations(bool flag) { fuse_activations_ = flag; }
    // Concat in place: a Conv (channel axis) or a re-padding Reshape (any other axis) whose result
    // only a Concat reads writes straight into its slice of the Concat's tensor, and a Concat
    // whose slices are all written that way is dropped from the sequence, where the reference
    // draws one full-output pass per input (nn/kernels/concat.cc:73-96). The producers' own
    // tensors are then not produced; GetOutputs on them fails with a message naming this
    // switch (default on; OGLE_FUSE_CONCATS=0 disables). Set before the first Run.
    void set_fuse_concats(bool flag) { fuse_concats_ = flag; }
    void set_fuse_residuals(bool flag) { fuse_residuals_ = flag; }
    int num_residuals() const { return num_residuals_; }
    // Launch tuning: after set-up every node may time variants of its launch that give identical results
    // and keep the fastest (convolutions on the tensor cores: the tile width). Default on; OGLE_TUNE=0
    // disables. Set before the first Run.
    void set_tune(bool flag) { tune_ = flag; }
    int num_placed() const { return num_placed_; }
    // Branch overlap: the captured graph keeps only the true data dependencies between
    // nodes, recorded over up to `n` streams, so that independent branches (the SSD heads
    // of one feature map against the layers that continue from it) may run side by side
    // and fill each other's partly empty last rounds. 1 = a linear chain in file order, as
    // the reference executes (fbo_session.cc:127-156). Default 4; OGLE_STREAMS overrides.
    // Eager runs and Profile() are always linear. Set before the graph is captured.
    void set_streams(int n);
    int streams() const { return streams_; }
    // Number of graph branches that did not continue the stream of a predecessor (0 = chain).
    int num_branches() const { return num_branches_; }
    // Nodes executed per Run (not pre-computed, not aliases).
    int num_active_kernels() const;
    // One eager pass with an event pair around every node; the per-node table the
    // reference's profiler prints (nn/profiler/profiler.cc:10-46).
    std::vector<NodeTiming> Profile(const NamedTensorList& inputs_cpu);
    // Bytes of device memory held by tensors of this session.
    size_t device_bytes() const { return device_bytes_; }

private:
    bool CheckKernelReady(const Kernel* kernel);
    void UpdateKernelReady(const Kernel* kernel);
    void UploadInputs(const NamedTensorList& inputs_cpu);
    void Finalize();
    void FuseSiblings();
    void FuseActivations();
    void FuseResiduals();
    void FuseConcats();
    void Execute();
    void DropGraph();
    void PlanStreams();
    void RecordSequence();

    Context* context_;
    OwnedKernelList kernels_;
    dlxnet::ModelProto model_;
    OwnedTensorList total_tensors_;
    bool finalized_ = false;
    bool graph_created_ = false;
    NamedIndex tensor_name_index_;
    std::vector<bool> ready_;
    std::vector<Kernel*> active_;       // the steady-state sequence
    bool allow_resized_ = false;
    IntList default_input_sizes_;
    bool use_graph_ = true;
    bool fuse_siblings_ = true;
    bool fuse_activations_ = true;
    bool fuse_concats_ = true;
    bool fuse_residuals_ = true;
    int num_residuals_ = 0;
    bool tune_ = true;
    int num_placed_ = 0;
    std::vector<bool> elided_;                // tensors no node produces any more (activation / concat fusion)
    std::vector<std::string> elided_why_;     // per tensor: the switch that keeps it
    int num_fused_ = 0;
    int eager_runs_ = 0;
    int streams_ = 4;
    int num_branches_ = 0;
    std::vector<int> lane_;                   // stream of each node of active_
    std::vector<std::vector<int>> waits_;     // nodes on other streams it must wait for
    std::vector<bool> signals_;               // some node on another stream waits for it
    std::vector<void*> side_streams_;         // streams 1..n-1 (stream 0 is the context's)
    std::vector<void*> events_;               // one per signalling node, plus fork / join
    CUgraphExec_st* graph_exec_ = nullptr;
    size_t device_bytes_ = 0;
    friend class Kernel;
};

}  // namespace ogle
#endif
