// C ABI over the C++ runtime (include/ogle_runtime.h). Every entry point catches
// FatalError (the runtime's stand-in for the reference's process abort) and
// reports it as a status code plus a thread-local message.
#include <cstring>
#include <string>

#include "detector.h"
#include "host_placement.h"
#include "stream_plan.h"
#include "fbo_session.h"
#include "kernel_registry.h"
#include "ogle_runtime.h"
#include <cuda_runtime.h>

namespace {
thread_local std::string g_error;

template <class F>
int guarded(F f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}
}  // namespace

struct OgleSession {
    std::unique_ptr<ogle::Context> context;   // null when borrowed from a detector
    ogle::FBOSession* session = nullptr;
    std::unique_ptr<ogle::FBOSession> owned;
};

struct OgleDetector {
    std::unique_ptr<ogle::Context> context;
    std::unique_ptr<ogle::Detector> detector;
    OgleSession session_view;
};

static ogle::NamedTensorList make_inputs(std::vector<std::unique_ptr<ogle::Tensor>>* keep, int n, const char* const* names,
                                         const float* const* data, const int* const* shapes, const int* ranks,
                                         const int* dformats) {
    ogle::NamedTensorList inputs;
    for (int i = 0; i < n; ++i) {
        ogle::IntList shape(shapes[i], shapes[i] + ranks[i]);
        keep->emplace_back(new ogle::Tensor(ogle::Tensor::DT_FLOAT, shape, const_cast<float*>(data[i]),
                                            ogle::DataFormat(dformats[i])));
        inputs.emplace_back(names[i], keep->back().get());
    }
    return inputs;
}

extern "C" {

const char* ogle_rt_last_error(void) { return g_error.c_str(); }

const char* ogle_rt_registered_kernels(void) {
    static thread_local std::string names;
    names.clear();
    for (const std::string& n : ogle::KernelRegistry::Global()->RegisteredNames()) names += n + "\n";
    return names.c_str();
}

OgleSession* ogle_session_create(int device, ogle_stream_t stream) {
    OgleSession* s = new OgleSession;
    if (guarded([&] {
            s->context.reset(new ogle::Context(device, stream));
            s->owned.reset(new ogle::FBOSession(s->context.get()));
            s->session = s->owned.get();
        }) != 0) {
        delete s;
        return nullptr;
    }
    return s;
}

void ogle_session_destroy(OgleSession* s) {
    if (!s) return;
    s->owned.reset();
    s->context.reset();
    delete s;
}

int ogle_session_set_option(OgleSession* s, const char* key, int value) {
    if (!s || !key) return -1;
    return guarded([&] {
        const std::string k(key);
        if (k == "math_mode") {
            OGLE_CHECK(value >= OGLE_MATH_FP32 && value <= OGLE_MATH_TF32X3) << "math_mode " << value;
            s->session->context()->set_math_mode(value);
        } else if (k == "use_graph") {
            s->session->set_use_graph(value != 0);
        } else if (k == "fuse_siblings") {
            s->session->set_fuse_siblings(value != 0);
        } else if (k == "fuse_activations") {
            s->session->set_fuse_activations(value != 0);
        } else if (k == "fuse_concats") {
            s->session->set_fuse_concats(value != 0);
        } else if (k == "fuse_residuals") {
            s->session->set_fuse_residuals(value != 0);
        } else if (k == "tune") {
            s->session->set_tune(value != 0);
        } else if (k == "streams") {
            s->session->set_streams(value);
        } else {
            OGLE_FATAL() << "unknown option " << k;
        }
    });
}

int ogle_session_load_graph_file(OgleSession* s, const char* path) {
    if (!s || !path) return -1;
    return guarded([&] { s->session->LoadGraph(std::string(path)); });
}

int ogle_session_load_graph_bytes(OgleSession* s, const void* data, size_t size) {
    if (!s || !data) return -1;
    return guarded([&] {
        dlxnet::ModelProto m;
        std::string err;
        OGLE_CHECK(dlxnet::ParseModel(data, size, &m, &err)) << "malformed dlx: " << err;
        s->session->LoadGraph(m);
    });
}

int ogle_session_run(OgleSession* s, int n, const char* const* names, const float* const* data, const int* const* shapes,
                     const int* ranks, const int* dformats) {
    if (!s || n < 0) return -1;
    return guarded([&] {
        std::vector<std::unique_ptr<ogle::Tensor>> keep;
        s->session->Run(make_inputs(&keep, n, names, data, shapes, ranks, dformats));
    });
}

int ogle_session_run_device(OgleSession* s, int n, const char* const* names, const float* const* data_device) {
    if (!s || n < 0) return -1;
    return guarded([&] {
        std::vector<std::pair<std::string, const float*>> in;
        for (int i = 0; i < n; ++i) in.emplace_back(names[i], data_device[i]);
        s->session->RunDevice(in);
    });
}

int ogle_session_synchronize(OgleSession* s) {
    if (!s) return -1;
    return guarded([&] { s->session->context()->MakeCurrent(); s->session->context()->Synchronize(); });
}

int ogle_session_tensor_info(OgleSession* s, const char* name, int* shape8, int* rank, int* dformat, void** device_ptr) {
    if (!s || !name) return -1;
    return guarded([&] {
        ogle::Tensor* t = s->session->FindTensorByName(name);
        OGLE_CHECK(t != nullptr) << "tensor " << name << " has not been produced yet";
        OGLE_CHECK_LE(t->shape().size(), 8u);
        if (rank) *rank = int(t->shape().size());
        if (shape8) for (size_t i = 0; i < t->shape().size(); ++i) shape8[i] = t->shape()[i];
        if (dformat) *dformat = int(t->dformat());
        if (device_ptr) *device_ptr = t->device();
    });
}

int ogle_session_get_output(OgleSession* s, const char* name, const char* dformat, float* out, size_t capacity) {
    if (!s || !name || !dformat || !out) return -1;
    return guarded([&] {
        ogle::Tensor* t = s->session->FindTensorByName(name);
        OGLE_CHECK(t != nullptr) << "tensor " << name << " has not been produced yet";
        const ogle::DataFormat f = ogle::StrToFormat(dformat);
        OGLE_CHECK_GE(capacity, ogle::CalcAllocatedSize1D(t->shape(), f)) << "output buffer too small for " << name;
        ogle::Tensor host(ogle::Tensor::DT_FLOAT, t->shape(), out, f);
        ogle::TensorList outs{&host};
        s->session->GetOutputs({name}, {dformat}, &outs);
    });
}

int ogle_session_num_active_kernels(OgleSession* s) { return s ? s->session->num_active_kernels() : -1; }
int ogle_session_num_placed(OgleSession* s) { return s ? s->session->num_placed() : -1; }
int ogle_session_num_residuals(OgleSession* s) { return s ? s->session->num_residuals() : -1; }
int ogle_session_num_branches(OgleSession* s) { return s ? s->session->num_branches() : -1; }
int ogle_session_graph_captured(OgleSession* s) { return s ? int(s->session->graph_captured()) : -1; }
size_t ogle_session_device_bytes(OgleSession* s) { return s ? s->session->device_bytes() : 0; }

int ogle_session_profile(OgleSession* s, int n, const char* const* names, const float* const* data, const int* const* shapes,
                         const int* ranks, const int* dformats, char* buf, size_t buf_size) {
    if (!s || !buf || buf_size == 0) return -1;
    return guarded([&] {
        std::vector<std::unique_ptr<ogle::Tensor>> keep;
        auto rows = s->session->Profile(make_inputs(&keep, n, names, data, shapes, ranks, dformats));
        std::string out;
        for (auto& r : rows) out += r.name + "\t" + r.type + "\t" + r.kernel + "\t" + std::to_string(r.ms) + "\n";
        OGLE_CHECK_LT(out.size(), buf_size) << "profile buffer too small";
        std::memcpy(buf, out.c_str(), out.size() + 1);
    });
}

OgleDetector* ogle_detector_create(int device, ogle_stream_t stream, const char* model_path, int mode, float score_thr,
                                   int top_k, float nms_thr, int math_mode, const char* input_name,
                                   const char* logits_name, const char* boxes_name, const char* anchors_name) {
    if (!model_path) return nullptr;
    OgleDetector* d = new OgleDetector;
    if (guarded([&] {
            d->context.reset(new ogle::Context(device, stream));
            if (math_mode >= 0) d->context->set_math_mode(math_mode);
            ogle::DetectorOptions o;
            o.model_name = model_path;
            o.mode = mode;
            o.score_threshold = score_thr;
            o.topk = top_k;
            o.nms_threshold = nms_thr;
            if (input_name) o.input_names = {input_name};
            if (logits_name) o.output_names[0] = logits_name;
            if (boxes_name) o.output_names[1] = boxes_name;
            if (anchors_name) o.output_names[2] = anchors_name;
            d->detector.reset(new ogle::Detector(o, d->context.get()));
            d->session_view.session = d->detector->session();
        }) != 0) {
        delete d;
        return nullptr;
    }
    return d;
}

void ogle_detector_destroy(OgleDetector* d) {
    if (!d) return;
    d->detector.reset();
    d->context.reset();
    delete d;
}

int ogle_detector_detect_async(OgleDetector* d, const float* images, int N, int H, int W) {
    if (!d || !images || N <= 0) return -1;
    return guarded([&] { d->detector->DetectAsync(images, N, H, W); });
}

int ogle_detector_detect_bgr8_async(OgleDetector* d, const unsigned char* const* images, const int* heights,
                                    const int* widths, int N, int H, int W, const float* mean_rgb) {
    if (!d) return -1;
    return guarded([&] { d->detector->DetectBGR8Async(images, heights, widths, N, H, W, mean_rgb); });
}

int ogle_detector_detect_device_async(OgleDetector* d, const float* images, int N, int H, int W, int copy_back) {
    if (!d || !images || N <= 0) return -1;
    return guarded([&] { d->detector->DetectDeviceAsync(images, N, H, W, copy_back != 0); });
}

int ogle_detector_wait(OgleDetector* d, float* score, int* anchor, int* cls, float* box, int* count) {
    if (!d) return -1;
    return guarded([&] {
        const ogle::DetectionBatch& r = d->detector->Wait();
        const size_t n = size_t(r.images) * r.rows;
        if (score) std::memcpy(score, r.score, n * 4);
        if (anchor) std::memcpy(anchor, r.anchor, n * 4);
        if (cls) std::memcpy(cls, r.cls, n * 4);
        if (box) std::memcpy(box, r.box, n * 16);
        if (count) std::memcpy(count, r.count, size_t(r.images) * r.counts_per_image * 4);
    });
}

int ogle_detector_info(OgleDetector* d, int* num_anchors, int* num_classes, int* rows, size_t* h2d, size_t* d2h) {
    if (!d) return -1;
    if (num_anchors) *num_anchors = d->detector->num_anchors();
    if (num_classes) *num_classes = d->detector->num_classes();
    if (rows) *rows = d->detector->rows();
    if (h2d) *h2d = d->detector->h2d_bytes();
    if (d2h) *d2h = d->detector->d2h_bytes();
    return 0;
}

OgleSession* ogle_detector_session(OgleDetector* d) { return d ? &d->session_view : nullptr; }

int ogle_host_bind_to_device(int device, int* numa_node, int* cpus_bound, int* memory_preferred) {
    const ogle::HostPlacement r = ogle::BindHostToDevice(device);
    if (numa_node) *numa_node = r.numa_node;
    if (cpus_bound) *cpus_bound = r.cpus_bound;
    if (memory_preferred) *memory_preferred = r.memory_preferred ? 1 : 0;
    return 0;
}

int ogle_rt_plan_streams(int n_nodes, int n_spans, const int* span_node, const unsigned long long* span_lo,
                         const unsigned long long* span_hi, const int* span_is_write, int streams, int* lane,
                         unsigned char* waits) {
    if (n_nodes < 0 || n_spans < 0 || (n_nodes && !lane) || (n_spans && (!span_node || !span_lo || !span_hi || !span_is_write)))
        return -1;
    std::vector<ogle::NodeAccess> nodes{size_t(n_nodes)};
    for (int i = 0; i < n_spans; ++i) {
        if (span_node[i] < 0 || span_node[i] >= n_nodes) return -1;
        ogle::NodeAccess& a = nodes[size_t(span_node[i])];
        (span_is_write[i] ? a.writes : a.reads).push_back(ogle::MemSpan{uintptr_t(span_lo[i]), uintptr_t(span_hi[i])});
    }
    const ogle::StreamPlan plan = ogle::PlanStreamsFor(nodes, streams);
    for (int i = 0; i < n_nodes; ++i) {
        lane[i] = plan.lane[size_t(i)];
        if (waits) {
            for (int j = 0; j < n_nodes; ++j) waits[size_t(i) * n_nodes + j] = 0;
            for (int j : plan.waits[size_t(i)]) waits[size_t(i) * n_nodes + j] = 1;
        }
    }
    return plan.branches;
}

void* ogle_host_alloc_pinned(size_t bytes) { return ogle::AllocPinnedHost(bytes); }
void ogle_host_free_pinned(void* p) { ogle::FreePinnedHost(p); }
size_t ogle_host_huge_page_bytes(const void* p) { return ogle::HugePageBytes(p); }

void* ogle_host_shared_open(const char* name, size_t bytes, int create, int pin) {
    if (!name) return nullptr;
    std::string err;
    void* p = ogle::OpenSharedHost(name, bytes, create != 0, pin != 0, &err);
    if (!p) g_error = err;
    return p;
}
void ogle_host_shared_close(void* p, int unlink) { ogle::CloseSharedHost(p, unlink != 0); }

int ogle_host_upload_async(void* dst_device, const void* src_host, size_t bytes, ogle_stream_t stream) {
    if (!dst_device || !src_host) return -1;
    const cudaError_t e = cudaMemcpyAsync(dst_device, src_host, bytes, cudaMemcpyHostToDevice, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { g_error = std::string("cudaMemcpyAsync: ") + cudaGetErrorString(e); return -3; }
    return 0;
}

int ogle_detector_use_result_buffers(OgleDetector* d, void* slot0, void* slot1, size_t bytes_each) {
    if (!d) return -1;
    return guarded([&] { d->detector->UseResultBuffers(slot0, slot1, bytes_each); });
}

int ogle_detector_result_layout(int mode, int num_classes, int top_k, int N, size_t* offsets6, int* rows, int* counts_per_image) {
    if (mode < 0 || mode > 1 || num_classes < 2 || top_k <= 0 || N <= 0 || !offsets6) return -1;
    const ogle::Detector::ResultLayout L = ogle::Detector::LayoutFor(mode, num_classes, top_k, N);
    offsets6[0] = L.score; offsets6[1] = L.anchor; offsets6[2] = L.cls; offsets6[3] = L.box; offsets6[4] = L.count;
    offsets6[5] = L.total;
    if (rows) *rows = L.rows;
    if (counts_per_image) *counts_per_image = L.counts_per_image;
    return 0;
}

int ogle_host_parse_cpulist(const char* text, int* cpus, int capacity) {
    if (!text) return -1;
    const std::vector<int> v = ogle::ParseCpuList(text);
    for (int i = 0; i < int(v.size()) && i < capacity; ++i)
        if (cpus) cpus[i] = v[size_t(i)];
    return int(v.size());
}

}  // extern "C"
