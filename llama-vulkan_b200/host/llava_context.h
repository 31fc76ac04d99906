// Process-level state: the model file, the CUDA context behind the C ABI, the
// layers and the read-only tensors shared by all sessions.  Counterpart of the
// reference's llava_context (llava_context.h:16-84); the Vulkan instance,
// device, queue, pools and pipeline cache become one lv_ctx.
#ifndef LLAVA_B200_CONTEXT_H
#define LLAVA_B200_CONTEXT_H

#include <mutex>
#include <string>
#include <vector>

#include "../../include/lv_b200.h"
#include "ggml_file.h"
#include "types.h"

class llava_context {
public:
    llava_context();
    ~llava_context();
    llava_context(const llava_context&) = delete;
    llava_context& operator=(const llava_context&) = delete;

    // Command-line entry point (llava_context.cpp:151-380 of the reference).
    int run(int argc, char** argv);
    // Opens the model, creates the device context and uploads all layers.
    bool open(const std::string& model_path, int device = 0);
    // Reads the model file only (header, vocabulary, tensor table) and creates no device context: enough for the
    // front end's session-independent requests; sessions cannot be created on such a context.
    bool open_model_only(const std::string& model_path);
    bool has_device() const { return lv_context != nullptr; }
    // Tensor-parallel open: this process is rank `rank` of `n_ranks` (one GPU each) and uploads
    // only its shard of every layer.  nccl_id: the 128 bytes of lv_comm_unique_id made by rank 0.
    bool open_sharded(const std::string& model_path, int device, u32 rank, u32 n_ranks, const u8* nccl_id);
    // Peer-memory all-reduce (lv_allreduce_add_f32 as one kernel): every rank makes a window and
    // its 64-byte IPC handle, the handles of all ranks are exchanged by the caller, then connected.
    bool peer_window_create(u8* handle64);
    bool peer_connect(const u8* handles);
    // true once the ranks' windows are connected: the all-reduces are then split between the
    // producing and the consuming GEMV instead of running as kernels of their own
    bool fused_exchange() const { return peers_connected && fused_exchange_enabled; }
    void set_fused_exchange(bool on) { fused_exchange_enabled = on; }
    u32 tp_rank() const { return rank_; }
    u32 tp_size() const { return n_ranks_; }

    lv_ctx* lv() const { return lv_context; }
    // the one device arena that holds every weight tensor of the model
    llava_device_memory* weights_memory() const { return shared_memory; }
    const ggml_file* get_model() const { return model; }
    std::vector<llava_layer*>& get_layers() { return layers; }
    bool upload_from_host(void* device_dst, const void* host_src, size_t bytes);
    bool signal_debug_on() const { return signal_debug; }
    int get_signal_fd() const { return sigfd; }
    u32 pop_signal(bool blocking = false) const;       // 0: none pending

    // read-only tensors shared by every session (the reference re-uploads the
    // last two per session, llava_session.cpp:73-78)
    llava_buffer* tok_embeddings = nullptr;
    llava_buffer* norm_w = nullptr;
    llava_buffer* output_w = nullptr;
    float* rope_table = nullptr;                        // [max_backlog][rot/2][2] cos/sin by distance

    u32 workgroup_size = 1024;       // kept for interface parity; kernel geometry is compile-time here
    u32 verbosity = 0;
    std::mutex queue_mutex;          // serialises sessions that share the stream

private:
    bool peers_connected = false;
    bool fused_exchange_enabled = true;
    bool setup_signal_handling();
    void close_all();
    ggml_file* model = nullptr;
    lv_ctx* lv_context = nullptr;
    llava_device_memory* shared_memory = nullptr;
    std::vector<llava_layer*> layers;
    bool signal_debug = false;
    int sigfd = -1;
    u32 rank_ = 0, n_ranks_ = 1;
};

#endif
