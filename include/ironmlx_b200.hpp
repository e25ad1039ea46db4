// C++ host mirror of the reference's layer surface for the MoE block, on top
// of the C ABI of ironmlx_b200.h (header-only; link libironmlx_b200.so and the
// CUDA runtime).  Names, fields and argument meaning follow the reference's
// Rust types so that a port of its call sites reads the same:
//
//   Array                       mlx/src/array.rs (here: a non-owning view of device memory)
//   Error / check               mlx/src/error.rs:17-54 (message of the failed call)
//   Linear                      mlx/src/nn/linear.rs:150-177 (dense, bf16)
//   QuantizedLinear             mlx/src/nn/linear.rs:13-63 (new, new_with_mode, forward_with_stream)
//   RMSNorm                     mlx/src/nn/norm.rs:11-24 (weight, eps, forward_with_stream -> fast::rms_norm)
//   MLP / Expert                mlx/src/nn/mlp.rs:12-33, mlx/src/nn/moe.rs:11-33
//   MoEMLP                      mlx/src/nn/moe.rs:39-183 (gate, experts, shared_expert,
//                               shared_expert_gate, num_experts_per_tok, norm_topk_prob,
//                               forward_with_stream)
//   ops::quantized_matmul, ops::dequantize   mlx/src/ops.rs:653-727
//
// Differences a port has to know: outputs are written into caller-provided
// arrays (no allocator here), the routed experts are held as the two fused
// checkpoint tensors (mlx/src/model/qwen35.rs:581-590) instead of a Vec of
// per-expert views, and the block keeps one device workspace per MoEMLP.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "ironmlx_b200.h"

namespace ironmlx {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

// Non-zero status -> exception carrying imx_last_error(), the analogue of `Error::Mlx`.
inline void check(int rc) {
    if (rc != IMX_OK) throw Error(rc, imx_last_error());
}
inline void check_cuda(cudaError_t e) {
    if (e != cudaSuccess) throw Error(IMX_ERR_CUDA, cudaGetErrorString(e));
}

enum class Dtype { Bfloat16, Float16, Float32, Uint32, Uint8, Int32 };

inline size_t dtype_size(Dtype d) {
    switch (d) {
        case Dtype::Bfloat16: case Dtype::Float16: return 2;
        case Dtype::Uint8: return 1;
        default: return 4;
    }
}

// View of a device tensor: pointer, shape, element type.  Owns nothing.
struct Array {
    void* ptr = nullptr;
    std::vector<int64_t> shape;
    Dtype dtype = Dtype::Bfloat16;

    Array() = default;
    Array(void* p, std::vector<int64_t> s, Dtype d) : ptr(p), shape(std::move(s)), dtype(d) {}
    int64_t size() const {
        int64_t n = 1;
        for (int64_t d : shape) n *= d;
        return n;
    }
    int64_t dim(int i) const { return shape[i < 0 ? (int)shape.size() + i : i]; }
    size_t nbytes() const { return (size_t)size() * dtype_size(dtype); }
};

inline int mode_id(const std::string& mode) {
    if (mode == "affine") return IMX_MODE_AFFINE;
    if (mode == "mxfp8") return IMX_MODE_MXFP8;
    if (mode == "nvfp4") return IMX_MODE_NVFP4;
    throw Error(IMX_ERR_INVALID, "unknown quantization mode '" + mode + "'");
}

// Device scratch of the layer calls: grown on demand, zero-filled (its first word is a device status word),
// one per host thread.
class Scratch {
public:
    Scratch() = default;
    Scratch(const Scratch&) = delete;
    Scratch& operator=(const Scratch&) = delete;
    ~Scratch() {
        if (ptr_) cudaFree(ptr_);
    }
    void* get(size_t need) {
        if (need > bytes_) {
            if (ptr_) check_cuda(cudaFree(ptr_));
            ptr_ = nullptr;
            bytes_ = 0;
            check_cuda(cudaMalloc(&ptr_, need));
            check_cuda(cudaMemset(ptr_, 0, need));
            bytes_ = need;
        }
        return ptr_;
    }
    size_t bytes() const { return bytes_; }
    static Scratch& local() {
        static thread_local Scratch s;
        return s;
    }

private:
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
};

namespace ops {

// x [M, in] (bf16) times a packed weight [out, in] (transpose = true) or [in, out] (false).
inline void quantized_matmul(const Array& x, const Array& w, const Array& scales, const Array* biases, bool transpose,
                             int group_size, int bits, const std::string& mode, Array& y, cudaStream_t stream = nullptr,
                             float global_scale = 1.f) {
    imx_qtensor q{w.ptr, scales.ptr, biases ? biases->ptr : nullptr, global_scale};
    const int in = (int)x.dim(-1), m = (int)(x.size() / in), n_out = (int)y.dim(-1);
    if (transpose) {     // the layers' form: on the expert kernels where they take the shape
        size_t need = 0;
        check(imx_quantized_matmul_scratch_bytes(m, n_out, in, group_size, bits, mode_id(mode), &need));
        Scratch& sc = Scratch::local();
        void* ws = sc.get(need);
        check(imx_quantized_matmul_ws(x.ptr, m, &q, n_out, in, group_size, bits, mode_id(mode), y.ptr, ws, sc.bytes(), stream));
        return;
    }
    check(imx_quantized_matmul(x.ptr, m, &q, n_out, in, 0, group_size, bits, mode_id(mode), y.ptr, stream));
}

// Packed weight [rows, in] -> dense bf16 / fp32 `out`.
inline void dequantize(const Array& w, const Array& scales, const Array* biases, int group_size, int bits,
                       const std::string& mode, Array& out, cudaStream_t stream = nullptr, float global_scale = 1.f) {
    imx_qtensor q{w.ptr, scales.ptr, biases ? biases->ptr : nullptr, global_scale};
    const int in = (int)out.dim(-1), rows = (int)(out.size() / in);
    check(imx_dequantize(&q, rows, in, group_size, bits, mode_id(mode), out.dtype == Dtype::Float32 ? 1 : (out.dtype == Dtype::Float16 ? 2 : 0), out.ptr,
                         stream));
}

}  // namespace ops

// Dense bf16 projection x . W^T (+ b) (mlx/src/nn/linear.rs:129-177); inside the block it is only a holder of
// its weight (router, shared-expert gate).
struct Linear {
    Array weight;                 // [out, in] bf16
    std::optional<Array> bias;    // [out] bf16
    explicit Linear(Array w = {}, std::optional<Array> b = std::nullopt) : weight(std::move(w)), bias(std::move(b)) {}
    void forward_with_stream(const Array& x, Array& y, cudaStream_t stream = nullptr) const {
        const int in = (int)weight.dim(1), n_out = (int)weight.dim(0);
        if (x.dim(-1) != in || y.dim(-1) != n_out) throw Error(IMX_ERR_INVALID, "Linear: shapes do not match the weight");
        check(imx_linear(x.ptr, (int)(x.size() / in), in, weight.ptr, n_out, bias ? bias->ptr : nullptr, y.ptr, stream));
    }
};

struct QuantizedLinear {
    Array weight, scales;
    std::optional<Array> biases;
    int group_size = 64, bits = 4;
    std::string mode = "affine";
    float global_scale = 1.f;

    static QuantizedLinear new_(Array weight, Array scales, Array biases, int group_size, int bits) {
        QuantizedLinear q;
        q.weight = std::move(weight);
        q.scales = std::move(scales);
        q.biases = std::move(biases);
        q.group_size = group_size;
        q.bits = bits;
        return q;
    }
    static QuantizedLinear new_with_mode(Array weight, Array scales, std::optional<Array> biases, int group_size, int bits,
                                         const std::string& mode, float global_scale = 1.f) {
        QuantizedLinear q;
        q.weight = std::move(weight);
        q.scales = std::move(scales);
        q.biases = std::move(biases);
        q.group_size = group_size;
        q.bits = bits;
        q.mode = mode;
        q.global_scale = global_scale;
        return q;
    }
    // y = quantized_matmul(x, w, scales, biases, transpose = true, group_size, bits, mode)
    void forward_with_stream(const Array& x, Array& y, cudaStream_t stream = nullptr) const {
        ops::quantized_matmul(x, weight, scales, biases ? &*biases : nullptr, true, group_size, bits, mode, y, stream,
                              global_scale);
    }
    imx_qtensor qtensor() const {
        return imx_qtensor{weight.ptr, scales.ptr, biases ? biases->ptr : nullptr, global_scale};
    }
};

struct RMSNorm {
    Array weight;   // [H] bf16
    float eps = 1e-6f;
    RMSNorm(Array w, float e) : weight(std::move(w)), eps(e) {}
    void forward_with_stream(const Array& x, Array& y, cudaStream_t stream = nullptr) const {
        const int h = (int)x.dim(-1);
        check(imx_rms_norm(x.ptr, (int)(x.size() / h), h, weight.ptr, eps, y.ptr, stream));
    }
};

// SwiGLU MLP: down(silu(gate(x)) * up(x)) (mlx/src/nn/mlp.rs:12-33); the shared expert of the block.  Also one
// routed expert (`Expert`, mlx/src/nn/moe.rs:11-33): its projections are then views into the fused tensors.
// forward_with_stream needs the gate and up rows as ONE [2I, .] tensor: adjacent views are used in place, separate
// tensors are stacked once into device memory the object owns.
struct MLP {
    QuantizedLinear gate_proj, up_proj, down_proj;

    MLP() = default;
    MLP(QuantizedLinear g, QuantizedLinear u, QuantizedLinear d)
        : gate_proj(std::move(g)), up_proj(std::move(u)), down_proj(std::move(d)) {}
    MLP(const MLP& o) : gate_proj(o.gate_proj), up_proj(o.up_proj), down_proj(o.down_proj) {}
    MLP& operator=(const MLP& o) {
        if (this != &o) {
            release();
            gate_proj = o.gate_proj;
            up_proj = o.up_proj;
            down_proj = o.down_proj;
        }
        return *this;
    }
    ~MLP() { release(); }

    void forward_with_stream(const Array& x, Array& y, cudaStream_t stream = nullptr) {
        const int hidden = (int)x.dim(-1), m = (int)(x.size() / hidden);
        imx_moe_config c{};
        c.hidden = hidden;
        c.num_experts = 1;
        c.top_k = 1;
        c.intermediate = (int)gate_proj.weight.dim(0);
        c.norm_topk_prob = 1;
        c.mode = mode_id(gate_proj.mode);
        c.bits = gate_proj.bits;
        c.group_size = gate_proj.group_size;
        const imx_qtensor gu = fused_gate_up(stream), dn = down_proj.qtensor();
        size_t need = 0;
        check(imx_expert_scratch_bytes(&c, m, &need));
        Scratch& sc = Scratch::local();
        void* ws = sc.get(need);
        check(imx_expert_forward(&c, &gu, &dn, x.ptr, m, y.ptr, ws, sc.bytes(), stream));
    }

private:
    static bool adjacent(const Array& a, const Array& b) { return (const char*)b.ptr == (const char*)a.ptr + a.nbytes(); }
    imx_qtensor fused_gate_up(cudaStream_t stream) {
        const bool has_b = gate_proj.biases.has_value();
        if (adjacent(gate_proj.weight, up_proj.weight) && adjacent(gate_proj.scales, up_proj.scales) &&
            (!has_b || adjacent(*gate_proj.biases, *up_proj.biases)))
            return gate_proj.qtensor();
        if (!own_[0]) {
            auto stack = [&](const Array& a, const Array& b, void** out) {
                check_cuda(cudaMalloc(out, a.nbytes() + b.nbytes()));
                check_cuda(cudaMemcpyAsync(*out, a.ptr, a.nbytes(), cudaMemcpyDeviceToDevice, stream));
                check_cuda(cudaMemcpyAsync((char*)*out + a.nbytes(), b.ptr, b.nbytes(), cudaMemcpyDeviceToDevice, stream));
            };
            stack(gate_proj.weight, up_proj.weight, &own_[0]);
            stack(gate_proj.scales, up_proj.scales, &own_[1]);
            if (has_b) stack(*gate_proj.biases, *up_proj.biases, &own_[2]);
        }
        return imx_qtensor{own_[0], own_[1], own_[2], gate_proj.global_scale};
    }
    void release() {
        for (void*& p : own_) {
            if (p) cudaFree(p);
            p = nullptr;
        }
    }
    void* own_[3] = {nullptr, nullptr, nullptr};
};
using Expert = MLP;

// All routed experts as the two fused checkpoint tensors: gate_up [E, 2I, .] (gate rows first), down [E, H, .].
struct FusedExperts {
    QuantizedLinear gate_up, down;
    int num_experts() const { return (int)gate_up.weight.dim(0); }
    int intermediate() const { return (int)(gate_up.weight.dim(1) / 2); }
};

class MoEMLP {
public:
    Linear gate;                              // router [E, H]
    FusedExperts experts;
    std::optional<MLP> shared_expert;
    std::optional<Linear> shared_expert_gate; // [1, H]
    int num_experts_per_tok = 1;
    bool norm_topk_prob = true;
    int path = IMX_PATH_AUTO;

    MoEMLP(Linear gate_, FusedExperts experts_, std::optional<MLP> shared_, std::optional<Linear> shared_gate_, int top_k,
           bool norm)
        : gate(std::move(gate_)), experts(std::move(experts_)), shared_expert(std::move(shared_)),
          shared_expert_gate(std::move(shared_gate_)), num_experts_per_tok(top_k), norm_topk_prob(norm) {}
    MoEMLP(const MoEMLP&) = delete;
    MoEMLP& operator=(const MoEMLP&) = delete;
    ~MoEMLP() {
        if (workspace_) cudaFree(workspace_);
    }

    imx_moe_config config() const {
        imx_moe_config c{};
        c.hidden = (int)gate.weight.dim(1);
        c.num_experts = experts.num_experts();
        c.top_k = num_experts_per_tok;
        c.intermediate = experts.intermediate();
        c.shared_intermediate = shared_expert ? (int)shared_expert->gate_proj.weight.dim(0) : 0;
        c.norm_topk_prob = norm_topk_prob ? 1 : 0;
        c.mode = mode_id(experts.gate_up.mode);
        c.bits = experts.gate_up.bits;
        c.group_size = experts.gate_up.group_size;
        c.path = path;
        return c;
    }
    imx_moe_weights weights() const {
        imx_moe_weights w{};
        w.router_w = gate.weight.ptr;
        w.gate_up = experts.gate_up.qtensor();
        w.down = experts.down.qtensor();
        if (shared_expert) {
            w.shared_gate_proj = shared_expert->gate_proj.qtensor();
            w.shared_up_proj = shared_expert->up_proj.qtensor();
            w.shared_down_proj = shared_expert->down_proj.qtensor();
            w.shared_expert_gate_w = shared_expert_gate ? shared_expert_gate->weight.ptr : nullptr;
        }
        return w;
    }

    // x: bf16 [B, L, H] (or [N, H]) -> y of the same shape; enqueued on `stream`, no host synchronisation.
    void forward_with_stream(const Array& x, Array& y, cudaStream_t stream = nullptr) {
        const imx_moe_config c = config();
        if (x.dtype != Dtype::Bfloat16 || y.dtype != Dtype::Bfloat16 || x.dim(-1) != c.hidden || y.size() != x.size())
            throw Error(IMX_ERR_INVALID, "MoEMLP: x and y must be bfloat16 arrays [.., hidden] of equal size");
        const int n = (int)(x.size() / c.hidden);
        const imx_moe_weights w = weights();
        ensure_workspace(c, n);
        check(imx_moe_forward(&c, &w, x.ptr, n, y.ptr, workspace_, workspace_bytes_, stream, nullptr));
    }

    // The MoE half of a decoder layer (mlx/src/model/qwen35.rs:271-276): y = h + forward(norm.forward(h)),
    // with the normalisation and the residual add fused into the block's first and last kernels.
    void forward_residual(const Array& h, const RMSNorm& norm, Array& y, cudaStream_t stream = nullptr) {
        const imx_moe_config c = config();
        if (h.dtype != Dtype::Bfloat16 || y.dtype != Dtype::Bfloat16 || h.dim(-1) != c.hidden || y.size() != h.size())
            throw Error(IMX_ERR_INVALID, "MoEMLP: h and y must be bfloat16 arrays [.., hidden] of equal size");
        const int n = (int)(h.size() / c.hidden);
        const imx_moe_weights w = weights();
        ensure_workspace(c, n);
        check(imx_moe_forward_residual(&c, &w, h.ptr, norm.weight.ptr, norm.eps, n, y.ptr, workspace_, workspace_bytes_,
                                       stream, nullptr));
    }

    // Device status word of the block's kernels (bounded waits that expired); throws if it is set.
    void check_status(cudaStream_t stream = nullptr) const {
        if (workspace_) check(imx_moe_status(workspace_, stream));
    }

private:
    void ensure_workspace(const imx_moe_config& c, int n) {
        size_t need = 0;
        check(imx_moe_workspace_bytes(&c, n, &need));
        if (need <= workspace_bytes_) return;
        if (workspace_) check_cuda(cudaFree(workspace_));
        workspace_ = nullptr;
        workspace_bytes_ = 0;
        check_cuda(cudaMalloc(&workspace_, need));
        check_cuda(cudaMemset(workspace_, 0, need));     // the status word starts at zero
        workspace_bytes_ = need;
    }
    void* workspace_ = nullptr;
    size_t workspace_bytes_ = 0;
};

}  // namespace ironmlx
