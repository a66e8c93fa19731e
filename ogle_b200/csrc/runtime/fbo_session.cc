#include "fbo_session.h"

#include <cuda_runtime.h>
#include <cstdlib>

#include "kernel_registry.h"
#include "stream_plan.h"

namespace ogle {

#define OGLE_RT_CUDA(call)                                                              \
    do {                                                                                \
        cudaError_t e_ = (call);                                                        \
        if (e_ != cudaSuccess) OGLE_FATAL() << #call << ": " << cudaGetErrorString(e_); \
    } while (0)

FBOSession::FBOSession(Context* context) : context_(context) {
    if (const char* g = std::getenv("OGLE_USE_GRAPH")) use_graph_ = std::atoi(g) != 0;
    if (const char* g = std::getenv("OGLE_FUSE_SIBLINGS")) fuse_siblings_ = std::atoi(g) != 0;
    if (const char* g = std::getenv("OGLE_FUSE_ACTIVATIONS")) fuse_activations_ = std::atoi(g) != 0;
    if (const char* g = std::getenv("OGLE_FUSE_CONCATS")) fuse_concats_ = std::atoi(g) != 0;
    if (const char* g = std::getenv("OGLE_FUSE_RESIDUALS")) fuse_residuals_ = std::atoi(g) != 0;
    if (const char* g = std::getenv("OGLE_TUNE")) tune_ = std::atoi(g) != 0;
    if (const char* g = std::getenv("OGLE_STREAMS")) set_streams(std::atoi(g));
}

FBOSession::~FBOSession() {
    context_->MakeCurrent();
    DropGraph();
    for (void* e : events_) cudaEventDestroy(reinterpret_cast<cudaEvent_t>(e));
    for (void* st : side_streams_) cudaStreamDestroy(reinterpret_cast<cudaStream_t>(st));
}

void FBOSession::set_streams(int n) {
    streams_ = n < 1 ? 1 : (n > 8 ? 8 : n);
    DropGraph();
}

void FBOSession::DropGraph() {
    if (graph_exec_) {
        cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(graph_exec_));
        graph_exec_ = nullptr;
    }
}

void FBOSession::set_use_graph(bool flag) {
    use_graph_ = flag;
    if (!flag) DropGraph();
}

void FBOSession::LoadGraph(const std::string& model_path) {
    dlxnet::ModelProto model;
    std::string err;
    OGLE_CHECK(dlxnet::ReadModelFromFile(model_path, &model, &err)) << "Load Graph " << model_path << " Failed: " << err;
    LoadGraph(model);
}

void FBOSession::LoadGraph(const dlxnet::ModelProto& model_proto) {
    // fbo_session.cc:77-124
    context_->MakeCurrent();
    DropGraph();
    model_ = model_proto;
    kernels_.clear();
    active_.clear();
    total_tensors_.clear();
    tensor_name_index_.clear();
    default_input_sizes_.clear();
    const dlxnet::GraphProto& graph = model_.graph;
    total_tensors_.resize(graph.tensor_names.size());
    for (size_t i = 0; i < graph.tensor_names.size(); ++i) tensor_name_index_[graph.tensor_names[i]] = int(i);

    for (const dlxnet::NodeProto& node : graph.node) {
        if (node.type == "Input") {
            const auto& dims = node.attr.input_attr.dims;
            OGLE_CHECK_GE(dims.size(), 2u);
            for (size_t i = dims.size() - 2; i < dims.size(); ++i) default_input_sizes_.push_back(dims[i]);
            continue;
        }
        Kernel* kernel = nullptr;
        KernelRegistry::Global()->CreateKernel(node.type, &kernel, context_);
        if (kernel == nullptr) OGLE_FATAL() << "unsupported kernel name " << node.type;
        std::unique_ptr<Kernel> owned(kernel);
        for (int64_t idx : node.input_index)
            OGLE_CHECK(idx >= 0 && idx < int64_t(total_tensors_.size())) << "node " << node.name << " input index " << idx;
        for (int64_t idx : node.output_index)
            OGLE_CHECK(idx >= 0 && idx < int64_t(total_tensors_.size())) << "node " << node.name << " output index " << idx;
        kernel->Setup(node, this);
        kernels_.emplace_back(std::move(owned));
    }
    finalized_ = false;
    graph_created_ = true;
    eager_runs_ = 0;
    device_bytes_ = 0;
}

void FBOSession::UploadInputs(const NamedTensorList& inputs_cpu) {
    for (const auto& in : inputs_cpu) {
        const Tensor* input_cpu = in.second;
        auto iter = tensor_name_index_.find(in.first);
        if (iter == tensor_name_index_.end()) OGLE_FATAL() << "tensor_name: " << in.first << " Cannot Find";
        const int input_index = iter->second;
        if (!finalized_) {
            total_tensors_[input_index].reset(new Tensor(Tensor::DT_FLOAT, input_cpu->shape(), Tensor::DEVICE_TEXTURE,
                                                         FormatToStride4(input_cpu->dformat())));
            device_bytes_ += total_tensors_[input_index]->AllocatedSize();
        }
        context_->CopyCPUTensorToDevice(input_cpu, total_tensors_[input_index].get());
    }
}

void FBOSession::Setup(const NamedTensorList& inputs_cpu) {
    OGLE_CHECK(graph_created_) << "No Graph Loaded!";
    context_->MakeCurrent();
    UploadInputs(inputs_cpu);
    if (!finalized_) Finalize();
}

void FBOSession::Finalize() {
    // fbo_session.cc:196-252
    ready_.assign(total_tensors_.size(), false);
    active_.clear();
    for (size_t i = 0; i < kernels_.size(); ++i) {
        Kernel* kernel = kernels_[i].get();
        kernel->input_tensors_.clear();
        kernel->output_tensors_.clear();
        for (int idx : kernel->input_tensor_indexes_) {
            Tensor* t = total_tensors_[idx].get();
            OGLE_CHECK(t != nullptr) << "input tensor is uninitialized of kernel index: " << i << " (" << kernel->kernel_name() << ")";
            kernel->input_tensors_.push_back(t);
        }
        kernel->SelectKernel(kernel->input_tensors_);
        TensorShapeList output_shapes;
        kernel->InferOutputShape(kernel->input_tensors_, output_shapes);
        OGLE_CHECK_GT(output_shapes.size(), 0u);
        OGLE_CHECK_LE(output_shapes.size(), kernel->output_tensor_indexes_.size());
        for (size_t j = 0; j < output_shapes.size(); ++j) {
            const DataFormat dformat = kernel->GetOutputDFormat(int(j));
            Tensor* out = nullptr;
            if (kernel->IsNoOp()) {
                // the output is the input's memory under a new shape
                out = new Tensor(output_shapes[j], dformat, kernel->input_tensors_[0]->device<float>());
            } else {
                out = new Tensor(Tensor::DT_FLOAT, output_shapes[j], Tensor::DEVICE_TEXTURE, dformat);
                device_bytes_ += out->AllocatedSize();
            }
            total_tensors_[kernel->output_tensor_indexes_[j]].reset(out);
            kernel->output_tensors_.push_back(out);
        }
        if (CheckKernelReady(kernel)) {
            // pre-compute: constants, weight re-layout, shape arithmetic
            kernel->Compute();
            UpdateKernelReady(kernel);
        } else if (!kernel->IsNoOp()) {
            active_.push_back(kernel);
        }
    }
    // short launches (small tensors: a few images per step) gain from overlapping each kernel's prologue with
    // its predecessor's tail, long ones lose a little: decided per session from the bytes its tensors hold
    ogle_cuda_set_overlapped_launches(device_bytes_ < (size_t(1) << 30) ? 1 : 0);
    if (fuse_siblings_) FuseSiblings();
    elided_.assign(total_tensors_.size(), false);
    elided_why_.assign(total_tensors_.size(), std::string());
    if (fuse_activations_) FuseActivations();
    num_residuals_ = 0;
    if (fuse_residuals_) FuseResiduals();
    num_placed_ = 0;
    if (fuse_concats_) FuseConcats();
    context_->Synchronize();
    if (tune_)
        for (Kernel* k : active_) k->Tune();
    context_->Synchronize();
    finalized_ = true;
}

void FBOSession::FuseSiblings() {
    // A later node may run early, at its sibling's place: it reads only what the sibling
    // reads, every tensor has its own memory, and its consumers still come after it.
    num_fused_ = 0;
    for (size_t i = 0; i < active_.size(); ++i) {
        for (size_t j = i + 1; j < active_.size(); ++j) {
            if (active_[j]->kernel_type() != active_[i]->kernel_type()) continue;
            if (!active_[i]->AbsorbSibling(active_[j])) continue;
            active_[i]->absorbed_.push_back(active_[j]);
            active_.erase(active_.begin() + long(j));
            ++num_fused_;
            break;      // pairs only
        }
    }
}

void FBOSession::FuseActivations() {
    // The consumer's work moves to its producer's place: it reads nothing else, and its own
    // output is read only by nodes that come after it.
    for (size_t i = 0; i < active_.size(); ++i) {
        Kernel* producer = active_[i];
        if (producer->output_tensor_indexes_.size() != 1 || producer->output_tensors_.size() != 1) continue;
        const int out_id = producer->output_tensor_indexes_[0];
        // every reader of the tensor, aliases (reshapes) and pre-computed nodes included
        Kernel* only = nullptr;
        int readers = 0;
        for (const auto& k : kernels_)
            for (int id : k->input_tensor_indexes_)
                if (id == out_id) { ++readers; only = k.get(); }
        if (readers != 1 || only->input_tensor_indexes_.size() != 1) continue;
        size_t j = i + 1;
        while (j < active_.size() && active_[j] != only) ++j;
        if (j == active_.size()) continue;
        if (!producer->AbsorbConsumer(only)) continue;
        producer->absorbed_.push_back(only);
        active_.erase(active_.begin() + long(j));
        elided_[size_t(out_id)] = true;
        elided_why_[size_t(out_id)] = "its only reader, an activation, runs in the producer's pass (session option "
                                      "fuse_activations = 0 or OGLE_FUSE_ACTIVATIONS=0 keeps it)";
        ++num_fused_;
    }
}

void FBOSession::FuseResiduals() {
    // An Add whose one operand is a convolution's result that nothing else reads, and whose other operand is
    // complete before that convolution runs, moves into the convolution's pass together with the activation the
    // Add may have taken over.
    auto readers = [&](int id) {
        int n = 0;
        for (const auto& k : kernels_)
            for (int in : k->input_tensor_indexes_) n += in == id;
        return n;
    };
    auto position = [&](const Kernel* k) {
        for (size_t i = 0; i < active_.size(); ++i)
            if (active_[i] == k) return long(i);
        return long(-1);
    };
    for (size_t j = 0; j < active_.size(); ++j) {
        Kernel* add = active_[j];
        int act; float lo, hi; Tensor* dst = nullptr;
        if (add->input_tensor_indexes_.size() != 2 || !add->AsResidualAdd(&act, &lo, &hi, &dst)) continue;
        for (int side = 0; side < 2; ++side) {
            const int conv_id = add->input_tensor_indexes_[size_t(side)], res_id = add->input_tensor_indexes_[size_t(1 - side)];
            if (conv_id == res_id || readers(conv_id) != 1 || elided_[size_t(conv_id)] || elided_[size_t(res_id)]) continue;
            Kernel* conv = nullptr;
            Kernel* res_producer = nullptr;
            for (const auto& k : kernels_) {
                if (k->output_tensor_indexes_.size() == 1 && k->output_tensor_indexes_[0] == conv_id) conv = k.get();
                for (int out : k->output_tensor_indexes_)
                    if (out == res_id) res_producer = k.get();
            }
            const long ci = conv ? position(conv) : -1;
            if (ci < 0 || ci >= long(j)) continue;
            if (res_producer) {
                // an alias (same-bytes reshape) has no place in the sequence of its own; keep those out
                if (res_producer->IsNoOp()) continue;
                const long ri = position(res_producer);
                if (ri >= ci) continue;                        // not there yet when the convolution runs
                if (ri < 0) {
                    bool absorbed = false;                   // its work may run inside another node, later than we know
                    for (Kernel* a : active_)
                        for (Kernel* b : a->absorbed_) absorbed = absorbed || b == res_producer;
                    if (absorbed) continue;
                }
            }
            if (!conv->AbsorbResidualAdd(add, total_tensors_[size_t(res_id)].get(), dst, act, lo, hi)) continue;
            conv->absorbed_.push_back(add);
            conv->extra_writes_.push_back(dst);
            active_.erase(active_.begin() + long(j));
            --j;
            elided_[size_t(conv_id)] = true;
            elided_why_[size_t(conv_id)] = "its only reader, a residual Add, runs in the convolution's pass (session option "
                                            "fuse_residuals = 0 or OGLE_FUSE_RESIDUALS=0 keeps it)";
            const int add_out = add->output_tensor_indexes_[0];
            if (total_tensors_[size_t(add_out)].get() != dst && !elided_[size_t(add_out)]) {
                elided_[size_t(add_out)] = true;
                elided_why_[size_t(add_out)] = elided_why_[size_t(conv_id)];
            }
            ++num_residuals_;
            break;
        }
    }
}

void FBOSession::FuseConcats() {
    // Readers of a tensor: every node that lists it as an input, pre-computed ones and aliases included.
    auto readers = [&](int id) {
        int n = 0;
        for (const auto& k : kernels_)
            for (int in : k->input_tensor_indexes_) n += in == id;
        return n;
    };
    // The node of the steady-state sequence that writes the memory behind tensor `id`: its producer, or
    // for an alias (identity transpose, same-bytes reshape) the producer of what it aliases, as long as
    // every tensor on the way has one reader.
    auto writer_of = [&](int id, std::vector<int>* chain) -> Kernel* {
        for (int hops = 0; hops < 8; ++hops) {
            if (readers(id) != 1 || elided_[size_t(id)]) return nullptr;
            chain->push_back(id);
            Kernel* producer = nullptr;
            for (const auto& k : kernels_)
                if (!k->output_tensor_indexes_.empty() && k->output_tensor_indexes_[0] == id) producer = k.get();
            if (!producer || producer->output_tensors_.size() != 1) return nullptr;
            if (!producer->IsNoOp()) {
                for (Kernel* a : active_)
                    if (a == producer) return producer;
                return nullptr;                       // pre-computed, or absorbed by a sibling
            }
            if (producer->input_tensor_indexes_.empty()) return nullptr;
            id = producer->input_tensor_indexes_[0];
        }
        return nullptr;
    };
    for (size_t c = 0; c < active_.size();) {
        Kernel* cat = active_[c];
        long outer, chunk, stride, offset;
        if (cat->output_tensors_.size() != 1 || !cat->ConcatPlacement(0, &outer, &chunk, &stride, &offset)) { ++c; continue; }
        size_t placed = 0;
        const size_t n_in = cat->input_tensor_indexes_.size();
        for (size_t i = 0; i < n_in; ++i) {
            if (!cat->ConcatPlacement(int(i), &outer, &chunk, &stride, &offset)) continue;
            std::vector<int> chain;
            Kernel* w = writer_of(cat->input_tensor_indexes_[i], &chain);
            if (!w || w == cat) continue;
            // the writer must come before the concat in the sequence (file order guarantees it)
            if (!w->PlaceOutput(cat->output_tensors_[0], outer, chunk, stride, offset)) continue;
            w->extra_writes_.push_back(cat->output_tensors_[0]);
            cat->InputPlaced(int(i));
            for (int id : chain) {
                elided_[size_t(id)] = true;
                elided_why_[size_t(id)] = "its producer writes straight into the Concat that reads it (session option "
                                          "fuse_concats = 0 or OGLE_FUSE_CONCATS=0 keeps it)";
            }
            ++placed;
            ++num_placed_;
        }
        if (placed == n_in) active_.erase(active_.begin() + long(c));     // nothing left to copy
        else ++c;
    }
}

bool FBOSession::CheckKernelReady(const Kernel* kernel) {
    if (kernel->ForceReady()) return true;
    for (int id : kernel->input_tensor_indexes_)
        if (!ready_[id]) return false;
    return true;
}

void FBOSession::UpdateKernelReady(const Kernel* kernel) {
    for (int id : kernel->output_tensor_indexes_) ready_[id] = true;
}

int FBOSession::num_active_kernels() const { return int(active_.size()); }

void FBOSession::Execute() {
    cudaStream_t s = reinterpret_cast<cudaStream_t>(context_->stream());
    if (graph_exec_) {
        OGLE_RT_CUDA(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(graph_exec_), s));
        return;
    }
    if (use_graph_ && eager_runs_ >= 1 && !active_.empty()) {
        // Everything a node needs was created by the eager pass; this pass only records.
        cudaGraph_t graph = nullptr;
        OGLE_RT_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
        try {
            RecordSequence();
        } catch (...) {
            context_->set_stream(reinterpret_cast<ogle_stream_t>(s));
            cudaStreamEndCapture(s, &graph);
            if (graph) cudaGraphDestroy(graph);
            throw;
        }
        OGLE_RT_CUDA(cudaStreamEndCapture(s, &graph));
        cudaGraphExec_t exec = nullptr;
        cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) OGLE_FATAL() << "cudaGraphInstantiate: " << cudaGetErrorString(e);
        graph_exec_ = reinterpret_cast<CUgraphExec_st*>(exec);
        OGLE_RT_CUDA(cudaGraphLaunch(exec, s));
        return;
    }
    for (Kernel* k : active_) k->Compute();
    ++eager_runs_;
}

// The stream plan of the steady-state sequence (stream_plan.h), from the memory every node
// touches: a reshape that aliases its input shares its span, and a node counts with the nodes
// it absorbed.
void FBOSession::PlanStreams() {
    const size_t n = active_.size();
    std::vector<NodeAccess> nodes(n);
    auto add = [](std::vector<MemSpan>& v, const Tensor* t) {
        if (!t || !t->device()) return;
        const uintptr_t lo = reinterpret_cast<uintptr_t>(t->device());
        v.push_back(MemSpan{lo, lo + uintptr_t(t->AllocatedSize())});
    };
    for (size_t i = 0; i < n; ++i) {
        std::vector<Kernel*> parts{active_[i]};
        for (Kernel* k : active_[i]->absorbed_) parts.push_back(k);
        for (Kernel* k : parts) {
            for (const Tensor* t : k->input_tensors_) add(nodes[i].reads, t);
            for (const Tensor* t : k->output_tensors_) add(nodes[i].writes, t);
            for (const Tensor* t : k->extra_writes_) add(nodes[i].writes, t);
        }
    }
    StreamPlan plan = PlanStreamsFor(nodes, streams_);
    lane_ = plan.lane;
    waits_ = plan.waits;
    signals_ = plan.signals;
    num_branches_ = plan.branches;
}

// Records the steady-state sequence on the capturing stream of the context and its side
// streams, as planned by PlanStreams.
void FBOSession::RecordSequence() {
    PlanStreams();
    cudaStream_t s0 = reinterpret_cast<cudaStream_t>(context_->stream());
    const int n = int(active_.size());
    bool linear = true;
    for (int l : lane_) linear = linear && l == 0;
    if (linear) {
        for (Kernel* k : active_) k->Compute();
        return;
    }
    while (int(side_streams_.size()) < streams_ - 1) {
        cudaStream_t st;
        OGLE_RT_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
        side_streams_.push_back(st);
    }
    const size_t n_events = size_t(n) + size_t(streams_) + 1;
    while (events_.size() < n_events) {
        cudaEvent_t e;
        OGLE_RT_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        events_.push_back(e);
    }
    auto event = [&](size_t i) { return reinterpret_cast<cudaEvent_t>(events_[i]); };
    auto stream = [&](int lane) { return lane == 0 ? s0 : reinterpret_cast<cudaStream_t>(side_streams_[size_t(lane - 1)]); };
    // fork: the side streams join the capture
    OGLE_RT_CUDA(cudaEventRecord(event(size_t(n)), s0));
    for (int l = 1; l < streams_; ++l) OGLE_RT_CUDA(cudaStreamWaitEvent(stream(l), event(size_t(n)), 0));
    struct Restore {
        Context* c; ogle_stream_t s;
        ~Restore() { c->set_stream(s); }
    } restore{context_, context_->stream()};
    for (int i = 0; i < n; ++i) {
        cudaStream_t ls = stream(lane_[size_t(i)]);
        for (int j : waits_[size_t(i)]) OGLE_RT_CUDA(cudaStreamWaitEvent(ls, event(size_t(j)), 0));
        context_->set_stream(reinterpret_cast<ogle_stream_t>(ls));
        active_[size_t(i)]->Compute();
        if (signals_[size_t(i)]) OGLE_RT_CUDA(cudaEventRecord(event(size_t(i)), ls));
    }
    // join: everything recorded on a side stream ends before the graph does
    for (int l = 1; l < streams_; ++l) {
        OGLE_RT_CUDA(cudaEventRecord(event(size_t(n + l)), stream(l)));
        OGLE_RT_CUDA(cudaStreamWaitEvent(s0, event(size_t(n + l)), 0));
    }
}

void FBOSession::Run(const NamedTensorList& inputs_cpu) {
    Setup(inputs_cpu);
    OGLE_CHECK(finalized_) << "Please Setup Session First";
    Execute();
}

void FBOSession::RunDevice(const std::vector<std::pair<std::string, const float*>>& inputs_device) {
    OGLE_CHECK(finalized_) << "RunDevice needs a session that Run or Setup has finalized";
    context_->MakeCurrent();
    cudaStream_t s = reinterpret_cast<cudaStream_t>(context_->stream());
    for (const auto& in : inputs_device) {
        Tensor* t = FindTensorByName(in.first);
        OGLE_CHECK(t != nullptr && in.second != nullptr);
        if (in.second != t->device<float>())
            OGLE_RT_CUDA(cudaMemcpyAsync(t->device(), in.second, t->AllocatedSize(), cudaMemcpyDeviceToDevice, s));
    }
    Execute();
}

std::vector<NodeTiming> FBOSession::Profile(const NamedTensorList& inputs_cpu) {
    Setup(inputs_cpu);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(context_->stream());
    std::vector<cudaEvent_t> ev(active_.size() + 1);
    for (auto& e : ev) OGLE_RT_CUDA(cudaEventCreate(&e));
    OGLE_RT_CUDA(cudaEventRecord(ev[0], s));
    for (size_t i = 0; i < active_.size(); ++i) {
        active_[i]->Compute();
        OGLE_RT_CUDA(cudaEventRecord(ev[i + 1], s));
    }
    OGLE_RT_CUDA(cudaStreamSynchronize(s));
    std::vector<NodeTiming> out;
    for (size_t i = 0; i < active_.size(); ++i) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
        out.push_back({active_[i]->kernel_name(), active_[i]->kernel_type(), active_[i]->kernel_fname(), ms});
    }
    for (auto& e : ev) cudaEventDestroy(e);
    return out;
}

void FBOSession::GetOutputs(const TensorNameList& output_names, const StringList& output_dformats, TensorList* outputs) {
    OGLE_CHECK_EQ(output_names.size(), output_dformats.size());
    context_->MakeCurrent();
    if (outputs->size() < output_names.size()) outputs->resize(output_names.size());
    for (size_t i = 0; i < output_names.size(); ++i) {
        Tensor* gpu_tensor = FindTensorByName(output_names[i]);
        OGLE_CHECK(gpu_tensor != nullptr) << "tensor " << output_names[i] << " was never produced";
        const int id = tensor_name_index_[output_names[i]];
        OGLE_CHECK(!(id < int(elided_.size()) && elided_[size_t(id)]))
            << "tensor " << output_names[i] << " is not materialised: " << elided_why_[size_t(id)];
        const DataFormat dformat = StrToFormat(output_dformats[i]);
        if (outputs->at(i) == nullptr)
            outputs->at(i) = new Tensor(Tensor::DT_FLOAT, gpu_tensor->shape(), Tensor::HOST_MEMORY, dformat);
        context_->CopyDeviceTensorToCPU(gpu_tensor, outputs->at(i));
    }
}

std::string FBOSession::DebugString() const {
    std::ostringstream ss;
    ss << "ModelProto: producer " << model_.producer_name << ", " << model_.graph.node.size() << " nodes, "
       << model_.graph.tensor_names.size() << " tensors\n";
    for (auto& k : kernels_) ss << k->DebugString() << "\n";
    return ss.str();
}

Tensor* FBOSession::FindTensorByName(const std::string& name) {
    auto iter = tensor_name_index_.find(name);
    if (iter == tensor_name_index_.end()) OGLE_FATAL() << "tensor_name: " << name << " Cannot Find";
    return FindTensorById(iter->second);
}

Tensor* FBOSession::FindTensorById(int id) {
    OGLE_CHECK_LT(id, int(total_tensors_.size()));
    return total_tensors_[id].get();
}

}  // namespace ogle
