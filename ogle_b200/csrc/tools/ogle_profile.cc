// Headless run / profile tool: the counterpart of the reference's nn/main.cc and
// nn/profile_main.cc (load a dlx, warm up, run num_iters times with read-back, print the
// per-node-type time table of nn/profiler/profiler.cc:10-46), without a window system.
//
//   ogle_profile model.dlx [num_iters] [--batch N] [--height H] [--width W] [--output NAME]
//                [--math fp32|tf32|tf32x3] [--verbose] [--json]
//
// The input is a tensor of ones named "input", NHWC [N,H,W,3] (profile_main.cc:78-82 uses
// 1x320x320x3; the default here is the model's Input node, else 1x300x300x3).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>

#include "fbo_session.h"

using namespace ogle;

int main(int argc, char** argv) {
    std::string model_path = "./demo.dlx", output = "cls_logits", math;
    int num_iters = 100, batch = 1, height = 0, width = 0;
    bool verbose = false, json = false;
    int positional = 0;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto next = [&](const char* flag) -> const char* {
            if (i + 1 >= argc) { std::fprintf(stderr, "%s needs a value\n", flag); std::exit(2); }
            return argv[++i];
        };
        if (a == "--batch") batch = std::atoi(next("--batch"));
        else if (a == "--height") height = std::atoi(next("--height"));
        else if (a == "--width") width = std::atoi(next("--width"));
        else if (a == "--output") output = next("--output");
        else if (a == "--math") math = next("--math");
        else if (a == "--verbose") verbose = true;
        else if (a == "--json") json = true;
        else if (positional == 0) { model_path = a; ++positional; }
        else if (positional == 1) { num_iters = std::atoi(a.c_str()); ++positional; }
        else { std::fprintf(stderr, "unexpected argument %s\n", a.c_str()); return 2; }
    }
    if (!math.empty()) {
        const char* v = math == "fp32" ? "0" : math == "tf32" ? "1" : math == "tf32x3" ? "2" : nullptr;
        if (!v) { std::fprintf(stderr, "--math takes fp32, tf32 or tf32x3\n"); return 2; }
        setenv("OGLE_MATH_MODE", v, 1);     // read when the context is created
    }
    try {
        std::unique_ptr<FBOSession> session(new FBOSession);
        session->LoadGraph(model_path);
        if (height <= 0 || width <= 0) {
            const IntList& d = session->default_input_sizes();
            height = d.size() == 2 ? d[0] : 300;
            width = d.size() == 2 ? d[1] : 300;
        }
        std::unique_ptr<Tensor> input(Tensor::Ones(Tensor::DT_FLOAT, {batch, height, width, 3}, dlxnet::TensorProto::NHWC));
        const NamedTensorList inputs{{"input", input.get()}};
        TensorList outputs_cpu;
        for (int i = 0; i < 3; ++i) {   // warming up (profile_main.cc:91-100)
            session->Run(inputs);
            session->GetOutputs({output}, {"ANY"}, &outputs_cpu);
        }
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < num_iters; ++i) {
            session->Run(inputs);
            session->GetOutputs({output}, {"ANY"}, &outputs_cpu);   // synchronises
        }
        const double total_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        // per node: one eager pass with an event pair around every node
        std::map<std::string, std::pair<double, int>> table;
        double device_ms = 0;
        const int passes = 5;
        for (int p = 0; p < passes; ++p)
            for (const NodeTiming& n : session->Profile(inputs)) {
                auto& e = table[verbose || n.type.empty() ? n.name : n.type];
                e.first += n.ms;
                e.second += 1;
                device_ms += n.ms;
            }
        if (json) {
            std::printf("{\"model\": \"%s\", \"batch\": %d, \"height\": %d, \"width\": %d, \"iters\": %d, "
                        "\"exec_ms_per_round\": %.4f, \"device_ms_per_round\": %.4f, \"graph\": %s, \"active_nodes\": %d, \"nodes\": {",
                        model_path.c_str(), batch, height, width, num_iters, total_ms / num_iters, device_ms / passes,
                        session->graph_captured() ? "true" : "false", session->num_active_kernels());
            bool first = true;
            for (const auto& it : table) {
                std::printf("%s\"%s\": {\"ms\": %.4f, \"count\": %d}", first ? "" : ", ", it.first.c_str(), it.second.first / passes,
                            it.second.second / passes);
                first = false;
            }
            std::printf("}}\n");
        } else {
            std::printf("ExecTimePerRound: %.3f ms (upload + %d nodes + read-back of %s, %s)\n", total_ms / num_iters,
                        session->num_active_kernels(), output.c_str(), session->graph_captured() ? "CUDA graph" : "eager");
            std::printf("----------------------profiler start------------------\n");
            std::printf("Node Type\tTime\tCount\n");
            for (const auto& it : table)
                std::printf("%s\t\t%.4fms\t\t%d\n", it.first.c_str(), it.second.first / passes, it.second.second / passes);
            std::printf("----------------------profiler end------------------\n");
        }
        for (Tensor* t : outputs_cpu) delete t;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ogle_profile: %s\n", e.what());
        return 1;
    }
    return 0;
}
