// hkv_engine_shim.hpp — a minimal stand-in for the host engine's op-dispatch boundary,
// used to exercise the adapter (hkv_register.hpp) without the engine itself.
//
// It models only what a registered op sees and what drives it, following the shapes of the
// reference engine (paths relative to the reference project root):
//   KernelFn(ExecContext&, const Command&)            src/engine.hpp:31-55
//   Command{op, output, inputs[], params{variant}}    src/command.hpp:28-96 — get<T>() returns the
//                                                     default unless the stored alternative is exactly T
//   TensorInfo{ptr, shape, dtype, size_bytes}         src/tensor.hpp:28-59
//   register_kernel overwrites an earlier entry       src/engine.cpp:40-45
//   device cache position scalars + update            src/engine.cpp:128-145
//   capture-once graph replay                         src/engine.cpp:151-269
// It is not a re-implementation of the engine: no memory pool, profiling, op registry
// singleton or non-capturable prefix handling.
#pragma once

#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <functional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <variant>
#include <vector>

namespace hkv_shim {

using OpTypeID = uint32_t;
namespace op {
inline OpTypeID ATTENTION_CACHED() { return 1; }
inline OpTypeID KV_CACHE_UPDATE() { return 2; }
inline OpTypeID ATTENTION_PREFILL_CACHED() { return 3; }
inline OpTypeID QK_NORM_ROPE() { return 4; }
}  // namespace op

enum class DType { INVALID, FP16, FP32, INT32 };
inline const char* dtype_name(DType d) {
    switch (d) {
        case DType::FP16: return "fp16";
        case DType::FP32: return "fp32";
        case DType::INT32: return "int32";
        default: return "invalid";
    }
}
inline size_t dtype_size(DType d) { return d == DType::FP16 ? 2 : 4; }

struct TensorInfo {
    void* ptr = nullptr;
    std::vector<uint32_t> shape;
    DType dtype = DType::INVALID;
    size_t size_bytes = 0;
    bool owns_memory = false;
};

using ParamValue = std::variant<bool, int32_t, int64_t, uint32_t, uint64_t, float, double, std::string>;

struct Command {
    OpTypeID op = 0;
    std::string output;
    std::vector<std::string> inputs;
    std::unordered_map<std::string, ParamValue> params;

    template <typename T>
    Command& set(const std::string& key, T value) {
        params[key] = ParamValue(std::move(value));
        return *this;
    }
    // Typed by exact alternative: a uint32_t parameter read as int32_t yields the default.
    template <typename T>
    T get(const std::string& key, T fallback = T{}) const {
        auto it = params.find(key);
        if (it == params.end()) return fallback;
        if (const T* v = std::get_if<T>(&it->second)) return *v;
        return fallback;
    }
    Command& in(std::initializer_list<std::string> names) {
        inputs.insert(inputs.end(), names);
        return *this;
    }
};

class CommandBuffer {
public:
    Command& add_op(OpTypeID id, const std::string& output = "") {
        cmds_.emplace_back();
        cmds_.back().op = id;
        cmds_.back().output = output;
        return cmds_.back();
    }
    // Same parameters and defaults as the engine's builders (src/command.cpp:154-184).
    void add_attention_cached(const std::string& dst, const std::string& q, const std::string& k_cache,
                              const std::string& v_cache, uint32_t num_heads, uint32_t num_kv_heads,
                              uint32_t head_dim, uint32_t seq_len, uint32_t max_seq_len,
                              uint32_t window_size = 0) {
        add_op(op::ATTENTION_CACHED(), dst)
            .in({q, k_cache, v_cache})
            .set("num_heads", num_heads)
            .set("num_kv_heads", num_kv_heads)
            .set("head_dim", head_dim)
            .set("scale", 1.0f / std::sqrt(static_cast<float>(head_dim)))
            .set("seq_len", seq_len)
            .set("max_seq_len", max_seq_len)
            .set("window_size", window_size);
    }
    void add_kv_cache_update(const std::string& k_cache, const std::string& v_cache,
                             const std::string& k_new, const std::string& v_new, uint32_t position,
                             uint32_t max_seq_len, uint32_t num_kv_heads, uint32_t head_dim,
                             uint32_t seq_len = 0) {
        add_op(op::KV_CACHE_UPDATE(), k_cache)
            .in({k_new, v_new, k_cache, v_cache})
            .set("position", position)
            .set("max_seq_len", max_seq_len)
            .set("num_kv_heads", num_kv_heads)
            .set("head_dim", head_dim)
            .set("seq_len", seq_len);
    }
    const std::vector<Command>& commands() const { return cmds_; }
    std::vector<Command>& commands() { return cmds_; }

private:
    std::vector<Command> cmds_;
};

struct ExecContext {
    cudaStream_t stream = nullptr;
    TensorInfo* output = nullptr;
    std::vector<TensorInfo*> inputs;
    TensorInfo* in(size_t i) const { return i < inputs.size() ? inputs[i] : nullptr; }
    size_t num_inputs() const { return inputs.size(); }
};

using KernelFn = std::function<void(ExecContext&, const Command&)>;

class TensorTable {
public:
    ~TensorTable() {
        for (auto& kv : map_)
            if (kv.second.owns_memory && kv.second.ptr) cudaFree(kv.second.ptr);
    }
    TensorInfo& allocate_and_register(const std::string& name, std::vector<uint32_t> shape, DType dt) {
        if (map_.count(name)) throw std::runtime_error("tensor already registered: " + name);
        TensorInfo t;
        t.shape = std::move(shape);
        t.dtype = dt;
        size_t n = 1;
        for (auto d : t.shape) n *= d;
        t.size_bytes = n * dtype_size(dt);
        if (cudaMalloc(&t.ptr, t.size_bytes) != cudaSuccess) throw std::runtime_error("cudaMalloc failed: " + name);
        cudaMemset(t.ptr, 0, t.size_bytes);
        t.owns_memory = true;
        return map_[name] = t;
    }
    TensorInfo& register_external(const std::string& name, void* ptr, std::vector<uint32_t> shape, DType dt) {
        if (map_.count(name)) throw std::runtime_error("tensor already registered: " + name);
        TensorInfo t;
        t.ptr = ptr;
        t.shape = std::move(shape);
        t.dtype = dt;
        size_t n = 1;
        for (auto d : t.shape) n *= d;
        t.size_bytes = n * dtype_size(dt);
        return map_[name] = t;
    }
    TensorInfo* get(const std::string& name) {
        auto it = map_.find(name);
        return it == map_.end() ? nullptr : &it->second;
    }
    TensorInfo& at(const std::string& name) {
        TensorInfo* t = get(name);
        if (!t) throw std::runtime_error("unknown tensor: " + name);
        return *t;
    }

private:
    std::unordered_map<std::string, TensorInfo> map_;
};

class Engine {
public:
    explicit Engine(cudaStream_t stream = nullptr) : stream_(stream) {}
    ~Engine() {
        invalidate_graph();
        if (d_cache_pos_) cudaFree(d_cache_pos_);
        if (d_total_seq_) cudaFree(d_total_seq_);
    }
    Engine(const Engine&) = delete;
    Engine& operator=(const Engine&) = delete;

    void register_kernel(OpTypeID id, KernelFn fn) { kernels_[id] = std::move(fn); }  // overwrites
    bool has_kernel(OpTypeID id) const { return kernels_.count(id) != 0; }
    TensorTable& tensors() { return tensors_; }
    cudaStream_t stream() const { return stream_; }

    void execute(const CommandBuffer& cb) {
        for (const auto& cmd : cb.commands()) run(cmd);
    }

    // Capture on the first call, replay afterwards; the command buffer is ignored once a
    // graph exists. Returns true when a graph was launched.
    bool execute_graph_replay(const CommandBuffer& cb) {
        if (graph_exec_) {
            cudaGraphLaunch(graph_exec_, stream_);
            return true;
        }
        cudaStreamSynchronize(stream_);
        cudaGetLastError();
        if (cudaStreamBeginCapture(stream_, cudaStreamCaptureModeGlobal) != cudaSuccess) {
            cudaGetLastError();
            execute(cb);
            return false;
        }
        bool ok = true;
        std::string what;
        for (const auto& cmd : cb.commands()) {
            try {
                run(cmd);
            } catch (const std::exception& e) {
                ok = false;
                what = e.what();
                break;
            }
        }
        cudaGraph_t graph = nullptr;
        const cudaError_t end = cudaStreamEndCapture(stream_, &graph);
        if (!ok || end != cudaSuccess || !graph) {
            if (graph) cudaGraphDestroy(graph);
            cudaGetLastError();
            last_capture_error_ = ok ? cudaGetErrorString(end) : what;
            execute(cb);
            return false;
        }
        if (cudaGraphInstantiate(&graph_exec_, graph, nullptr, nullptr, 0) != cudaSuccess) {
            cudaGraphDestroy(graph);
            graph_exec_ = nullptr;
            cudaGetLastError();
            execute(cb);
            return false;
        }
        graph_ = graph;
        cudaGraphLaunch(graph_exec_, stream_);
        return true;
    }
    void invalidate_graph() {
        if (graph_exec_) cudaGraphExecDestroy(graph_exec_);
        if (graph_) cudaGraphDestroy(graph_);
        graph_exec_ = nullptr;
        graph_ = nullptr;
    }
    bool graph_ready() const { return graph_exec_ != nullptr; }
    const std::string& last_capture_error() const { return last_capture_error_; }

    void alloc_device_cache_pos() {
        if (d_cache_pos_) return;
        cudaMalloc(&d_cache_pos_, sizeof(int32_t));
        cudaMalloc(&d_total_seq_, sizeof(int32_t));
        cudaMemset(d_cache_pos_, 0, sizeof(int32_t));
        cudaMemset(d_total_seq_, 0, sizeof(int32_t));
    }
    void update_device_cache_pos(int32_t cache_pos, int32_t seq_len) {
        if (!d_cache_pos_) alloc_device_cache_pos();
        h_pos_[0] = cache_pos;
        h_pos_[1] = cache_pos + seq_len;
        cudaMemcpyAsync(d_cache_pos_, &h_pos_[0], sizeof(int32_t), cudaMemcpyHostToDevice, stream_);
        cudaMemcpyAsync(d_total_seq_, &h_pos_[1], sizeof(int32_t), cudaMemcpyHostToDevice, stream_);
    }
    int32_t* device_cache_pos() const { return d_cache_pos_; }
    int32_t* device_total_seq() const { return d_total_seq_; }
    bool has_device_cache_pos() const { return d_cache_pos_ != nullptr; }
    void sync() { cudaStreamSynchronize(stream_); }

private:
    void run(const Command& cmd) {
        auto it = kernels_.find(cmd.op);
        if (it == kernels_.end()) throw std::runtime_error("no kernel registered for op");
        ExecContext ctx;
        ctx.stream = stream_;
        ctx.output = cmd.output.empty() ? nullptr : tensors_.get(cmd.output);
        for (const auto& name : cmd.inputs) ctx.inputs.push_back(tensors_.get(name));
        it->second(ctx, cmd);
    }

    cudaStream_t stream_;
    TensorTable tensors_;
    std::unordered_map<OpTypeID, KernelFn> kernels_;
    cudaGraph_t graph_ = nullptr;
    cudaGraphExec_t graph_exec_ = nullptr;
    std::string last_capture_error_;
    int32_t* d_cache_pos_ = nullptr;
    int32_t* d_total_seq_ = nullptr;
    int32_t h_pos_[2] = {0, 0};
};

}  // namespace hkv_shim
