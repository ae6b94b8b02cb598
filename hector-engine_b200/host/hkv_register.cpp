// hkv_register.cpp — ContextPool: one hkv_ctx per geometry, status codes -> exceptions.
#include "hkv_register.hpp"

namespace hkv {

ContextPool::~ContextPool() {
    for (auto& kv : ctxs_) hkv_ctx_destroy(kv.second);
}

hkv_ctx* ContextPool::get(const hkv_geometry& g) {
    const Key key{g.batch, g.num_heads, g.num_kv_heads, g.head_dim, g.slots, g.window_size, g.layout,
                  (long long)g.batch_stride_elems, g.max_seq_new, g.flags};
    auto it = ctxs_.find(key);
    if (it != ctxs_.end()) return it->second;
    hkv_ctx* c = nullptr;
    const int st = hkv_ctx_create(&c, &g);
    if (st != HKV_OK) {
        std::string msg = std::string("hkv_ctx_create: ") + hkv_status_string(st);
        if (c) {
            msg += std::string(" (") + hkv_ctx_last_error(c) + ")";
            hkv_ctx_destroy(c);
        }
        throw std::runtime_error(msg);
    }
    ctxs_[key] = c;
    return c;
}

void ContextPool::check(hkv_ctx* c, int status, const char* op) {
    if (status == HKV_OK) return;
    throw std::runtime_error(std::string(op) + ": " + hkv_status_string(status) + " (" +
                             hkv_ctx_last_error(c) + ")");
}

}  // namespace hkv
