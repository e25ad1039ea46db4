// Drives the C++ host mirror (include/ironmlx_b200.hpp) the way a port of the
// reference's qwen35.rs would: builds a MoEMLP from the fused checkpoint
// tensors, calls forward_with_stream and QuantizedLinear::forward_with_stream,
// and writes the results for the Python test to compare with the ctypes path.
//
//   mirror_main <dir>
// <dir>/meta.txt holds: tokens hidden experts top_k intermediate shared norm bits group
// <dir>/<name>.bin are raw tensors; outputs go to <dir>/y.bin, <dir>/yq.bin and <dir>/yt.bin.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

#include "ironmlx_b200.hpp"

using namespace ironmlx;

static std::vector<char> read_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::vector<char> b((size_t)f.tellg());
    f.seekg(0);
    f.read(b.data(), (std::streamsize)b.size());
    return b;
}

struct DeviceBuffers {
    std::vector<void*> all;
    ~DeviceBuffers() {
        for (void* p : all) cudaFree(p);
    }
    void* upload(const std::string& path, size_t expect) {
        const std::vector<char> h = read_file(path);
        if (h.size() != expect) throw std::runtime_error(path + ": unexpected size");
        void* d = nullptr;
        check_cuda(cudaMalloc(&d, h.size()));
        check_cuda(cudaMemcpy(d, h.data(), h.size(), cudaMemcpyHostToDevice));
        all.push_back(d);
        return d;
    }
    void* alloc(size_t n) {
        void* d = nullptr;
        check_cuda(cudaMalloc(&d, n));
        all.push_back(d);
        return d;
    }
};

int main(int argc, char** argv) {
    if (argc != 2) {
        std::fprintf(stderr, "usage: mirror_main <dir>\n");
        return 2;
    }
    const std::string dir = argv[1];
    try {
        long n, H, E, k, I, Is, norm, bits, group;
        {
            std::ifstream m(dir + "/meta.txt");
            if (!(m >> n >> H >> E >> k >> I >> Is >> norm >> bits >> group)) throw std::runtime_error("bad meta.txt");
        }
        DeviceBuffers dev;
        auto packed = [&](long rows, long in) { return (size_t)rows * in * bits / 8; };
        auto scale_b = [&](long rows, long in) { return (size_t)rows * (in / group) * 2; };
        auto qlin = [&](const std::string& name, std::vector<int64_t> lead, long rows, long in) {
            std::vector<int64_t> ws = lead, ss = lead;
            ws.push_back(rows); ws.push_back(in * bits / 32);
            ss.push_back(rows); ss.push_back(in / group);
            long mult = 1;
            for (int64_t d : lead) mult *= d;
            Array w(dev.upload(dir + "/" + name + "_w.bin", packed(rows, in) * mult), ws, Dtype::Uint32);
            Array s(dev.upload(dir + "/" + name + "_s.bin", scale_b(rows, in) * mult), ss, Dtype::Bfloat16);
            Array b(dev.upload(dir + "/" + name + "_b.bin", scale_b(rows, in) * mult), ss, Dtype::Bfloat16);
            return QuantizedLinear::new_(w, s, b, (int)group, (int)bits);
        };
        Linear gate(Array(dev.upload(dir + "/router_w.bin", (size_t)E * H * 2), {E, H}, Dtype::Bfloat16));
        FusedExperts experts{qlin("gate_up", {E}, 2 * I, H), qlin("down", {E}, H, I)};
        std::optional<MLP> shared;
        std::optional<Linear> shared_gate;
        if (Is > 0) {
            shared = MLP{qlin("shared_gate", {}, Is, H), qlin("shared_up", {}, Is, H), qlin("shared_down", {}, H, Is)};
            shared_gate = Linear(Array(dev.upload(dir + "/shared_expert_gate.bin", (size_t)H * 2), {1, H}, Dtype::Bfloat16));
        }
        MoEMLP moe(gate, experts, shared, shared_gate, (int)k, norm != 0);

        Array x(dev.upload(dir + "/x.bin", (size_t)n * H * 2), {1, n, H}, Dtype::Bfloat16);
        Array y(dev.alloc((size_t)n * H * 2), {1, n, H}, Dtype::Bfloat16);
        cudaStream_t stream;
        check_cuda(cudaStreamCreate(&stream));
        moe.forward_with_stream(x, y, stream);
        moe.forward_with_stream(x, y, stream);          // the workspace is reused
        check_cuda(cudaStreamSynchronize(stream));
        moe.check_status(stream);
        std::vector<char> hy((size_t)n * H * 2);
        check_cuda(cudaMemcpy(hy.data(), y.ptr, hy.size(), cudaMemcpyDeviceToHost));
        std::ofstream(dir + "/y.bin", std::ios::binary).write(hy.data(), (std::streamsize)hy.size());

        // QuantizedLinear::forward_with_stream on the first expert's down projection: [n, I] -> [n, H]
        QuantizedLinear down0 = experts.down;
        down0.weight.shape = {H, I * bits / 32};
        Array xq(dev.upload(dir + "/xq.bin", (size_t)n * I * 2), {n, I}, Dtype::Bfloat16);
        Array yq(dev.alloc((size_t)n * H * 2), {n, H}, Dtype::Bfloat16);
        down0.forward_with_stream(xq, yq, stream);
        check_cuda(cudaStreamSynchronize(stream));
        std::vector<char> hq((size_t)n * H * 2);
        check_cuda(cudaMemcpy(hq.data(), yq.ptr, hq.size(), cudaMemcpyDeviceToHost));
        std::ofstream(dir + "/yq.bin", std::ios::binary).write(hq.data(), (std::streamsize)hq.size());

        // decoder-layer tail: y = h + MoE(rms_norm(h)) with the norm weight from <dir>/ln_w.bin
        RMSNorm post_ln(Array(dev.upload(dir + "/ln_w.bin", (size_t)H * 2), {H}, Dtype::Bfloat16), 1e-6f);
        Array yt(dev.alloc((size_t)n * H * 2), {1, n, H}, Dtype::Bfloat16);
        moe.forward_residual(x, post_ln, yt, stream);
        check_cuda(cudaStreamSynchronize(stream));
        moe.check_status(stream);
        std::vector<char> ht((size_t)n * H * 2);
        check_cuda(cudaMemcpy(ht.data(), yt.ptr, ht.size(), cudaMemcpyDeviceToHost));
        std::ofstream(dir + "/yt.bin", std::ios::binary).write(ht.data(), (std::streamsize)ht.size());

        // MLP::forward_with_stream (the shared expert: three separate tensors, stacked once) and the dense router
        // Linear::forward_with_stream on the same tokens
        if (Is > 0) {
            MLP mlp = *shared;
            Array x2(x.ptr, {n, H}, Dtype::Bfloat16);
            Array ym(dev.alloc((size_t)n * H * 2), {n, H}, Dtype::Bfloat16);
            mlp.forward_with_stream(x2, ym, stream);
            Array yl(dev.alloc((size_t)n * E * 2), {n, E}, Dtype::Bfloat16);
            gate.forward_with_stream(x2, yl, stream);
            check_cuda(cudaStreamSynchronize(stream));
            std::vector<char> hm((size_t)n * H * 2), hl((size_t)n * E * 2);
            check_cuda(cudaMemcpy(hm.data(), ym.ptr, hm.size(), cudaMemcpyDeviceToHost));
            check_cuda(cudaMemcpy(hl.data(), yl.ptr, hl.size(), cudaMemcpyDeviceToHost));
            std::ofstream(dir + "/ym.bin", std::ios::binary).write(hm.data(), (std::streamsize)hm.size());
            std::ofstream(dir + "/yl.bin", std::ios::binary).write(hl.data(), (std::streamsize)hl.size());
        }

        // error convention: a wrong shape must surface as ironmlx::Error with the library's message
        bool threw = false;
        try {
            Array bad(x.ptr, {1, n, H + 16}, Dtype::Bfloat16);
            moe.forward_with_stream(bad, y, stream);
        } catch (const Error& e) {
            threw = e.code == IMX_ERR_INVALID;
        }
        if (!threw) throw std::runtime_error("a wrong shape was accepted");
        check_cuda(cudaStreamDestroy(stream));
        std::puts("mirror ok");
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "mirror_main: %s\n", e.what());
        return 1;
    }
}
