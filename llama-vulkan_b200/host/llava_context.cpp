#include "llava_context.h"

#include <signal.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <sys/poll.h>
#include <sys/signalfd.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <new>
#include <thread>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>

#include "llava_buffer.h"
#include "llava_device_memory.h"
#include "llava_layer.h"
#include "llava_session.h"
#include "server/tlv_server.h"
#include "synth_ggjt.h"

using namespace std;

llava_context::llava_context() = default;

llava_context::~llava_context() { close_all(); }

void llava_context::close_all() {
    for (llava_layer* l : layers) delete l;
    layers.clear();
    delete tok_embeddings;
    delete norm_w;
    delete output_w;
    tok_embeddings = norm_w = output_w = nullptr;
    if (rope_table && lv_context) lv_arena_free(lv_context, rope_table);
    rope_table = nullptr;
    delete shared_memory;
    shared_memory = nullptr;
    if (lv_context) lv_ctx_destroy(lv_context);
    lv_context = nullptr;
    rank_ = 0;
    n_ranks_ = 1;
    delete model;
    model = nullptr;
    if (sigfd >= 0) ::close(sigfd);
    sigfd = -1;
}

bool llava_context::upload_from_host(void* device_dst, const void* host_src, size_t bytes) {
    return lv_upload(lv_context, device_dst, host_src, bytes) == LV_OK;
}

bool llava_context::open_sharded(const string& model_path, int device, u32 rank, u32 n_ranks, const u8* nccl_id) {
    if (n_ranks == 0 || rank >= n_ranks || (n_ranks > 1 && nccl_id == nullptr)) return false;
    rank_ = rank;
    n_ranks_ = n_ranks;
    if (!open(model_path, device)) return false;
    if (n_ranks > 1 && lv_comm_init_rank(lv_context, nccl_id, int(n_ranks), int(rank)) != LV_OK) {
        cerr << "[!] cannot create the communicator: " << lv_last_error_string() << endl;
        return false;
    }
    return true;
}

bool llava_context::peer_window_create(u8* handle64) {
    if (lv_context == nullptr || model == nullptr) return false;
    return lv_peer_window_create(lv_context, int(n_ranks_), model->get_header().dim * llava_session::max_batch_limit, handle64) == LV_OK;
}

bool llava_context::peer_connect(const u8* handles) {
    peers_connected = lv_context != nullptr && lv_peer_connect(lv_context, int(rank_), handles) == LV_OK;
    return peers_connected;
}

bool llava_context::open_model_only(const string& model_path) {
    close_all();
    model = new ggml_file(model_path.c_str());
    return model->is_open();
}

bool llava_context::open(const string& model_path, int device) {
    const u32 keep_rank = rank_, keep_ranks = n_ranks_;
    close_all();
    rank_ = keep_rank;
    n_ranks_ = keep_ranks;
    model = new ggml_file(model_path.c_str());
    if (!model->is_open()) return false;
    const ggml_header& h = model->get_header();
    if (h.n_heads % n_ranks_ != 0 || (h.dim / 32) % n_ranks_ != 0 || (model->get_ff_size() / 32) % n_ranks_ != 0 ||
        model->get_ff_size() % (2 * n_ranks_) != 0) {
        cerr << "[!] heads, dim and ff must divide evenly over " << n_ranks_ << " ranks" << endl;
        return false;
    }
    // the kernels are specialised for the reference's geometries (llava_session.cpp:357-375:
    // dim 4096 or 5120, ff 11008 or 13824) and for heads of 128
    if (h.rot != 128 || h.dim % 256 != 0 || model->get_ff_size() % 256 != 0) {
        cerr << "[!] unsupported geometry: need head size 128 and dim, ff multiples of 256" << endl;
        return false;
    }
    if (lv_ctx_create(device, &lv_context) != LV_OK) {
        cerr << "[!] cannot create the CUDA context: " << lv_last_error_string() << endl;
        return false;
    }
    const ggml_data_descriptor* emb = model->find_buffer_descriptor("tok_embeddings");
    const ggml_data_descriptor* norm = model->find_buffer_descriptor("norm");
    const ggml_data_descriptor* out = model->find_buffer_descriptor("output");
    if (!emb || !norm || !out) {
        cerr << "[!] tok_embeddings / norm / output missing from the model" << endl;
        return false;
    }
    shared_memory = new llava_device_memory(this);
    tok_embeddings = new llava_buffer(this, *emb, shared_memory);
    norm_w = new llava_buffer(this, *norm, shared_memory);
    output_w = new llava_buffer(this, *out, shared_memory);
    if (norm_w->type != ggml_value_type::f32 || !output_w->weight_buffer_is_quantised() || emb->shape1 != h.vocab_size ||
        !(tok_embeddings->weight_buffer_is_quantised() || tok_embeddings->type == ggml_value_type::f32)) {
        cerr << "[!] unsupported tensor types for tok_embeddings / norm / output" << endl;
        return false;
    }

    void* table = nullptr;
    if (lv_arena_create(lv_context, size_t(max_backlog_size) * h.rot * sizeof(float), &table) != LV_OK) return false;
    rope_table = static_cast<float*>(table);
    if (lv_rope_table_build(lv_context, rope_table, max_backlog_size, h.rot) != LV_OK) return false;

    layers.reserve(h.n_layers);
    for (u32 i = 0; i < h.n_layers; ++i) {
        layers.push_back(new llava_layer(this, i));
        if (!layers.back()->is_valid()) return false;
    }
    // every tensor has registered its size: one allocation for the whole model
    if (!shared_memory->freeze()) return false;
    if (!tok_embeddings->load_to_gpu() || !norm_w->load_to_gpu() || !output_w->load_to_gpu()) return false;
    for (llava_layer* l : layers) {
        if (sigfd >= 0 && pop_signal()) return false;
        if (!l->freeze_storage() || !l->load_to_gpu()) {
            cerr << "[!] cannot upload layer " << l->layer_id << ": " << lv_last_error_string() << endl;
            return false;
        }
    }
    return true;
}

bool llava_context::setup_signal_handling() {
    if (signal_debug) return true;
    sigset_t mask;
    sigemptyset(&mask);
    for (int s : {SIGINT, SIGQUIT, SIGHUP, SIGTERM}) sigaddset(&mask, s);
    if (sigprocmask(SIG_BLOCK, &mask, nullptr) < 0) return false;
    sigfd = signalfd(-1, &mask, SFD_NONBLOCK | SFD_CLOEXEC);
    return sigfd >= 0;
}

u32 llava_context::pop_signal(bool blocking) const {
    if (sigfd < 0) return 0;
    if (blocking) {
        pollfd p{sigfd, POLLIN, 0};
        ::poll(&p, 1, -1);
    }
    signalfd_siginfo info{};
    const ssize_t r = ::read(sigfd, &info, sizeof info);
    return r == ssize_t(sizeof info) ? info.ssi_signo : 0;
}

namespace {
bool streq(const char* a, const char* b) { return strcmp(a, b) == 0; }

bool read_token_file(const string& path, vector<u32>* out) {
    ifstream in(path);
    if (!in) return false;
    u64 v;
    while (in >> v) out->push_back(u32(v));
    return !out->empty();
}

// What the ranks of `--gpus N` (one forked process per GPU) share: rank 0's communicator id and every rank's
// peer-window handle, in an anonymous shared mapping made before the fork.
struct tp_rendezvous {
    std::atomic<u32> id_ready, handles_ready, connected, failed, done;
    u8 nccl_id[128];
    u8 handles[8][64];
};

// Waits until `counter` reaches `target`; false after two minutes or when a rank reported a failure.
bool rendezvous_wait(const tp_rendezvous* rv, const std::atomic<u32>& counter, u32 target) {
    const auto t0 = std::chrono::steady_clock::now();
    while (counter.load(std::memory_order_acquire) < target) {
        if (rv->failed.load(std::memory_order_acquire)) return false;
        if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(120)) return false;
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    return true;
}
}  // namespace

// Flags of the reference (llava_context.cpp:163-200) that still mean something, plus the
// ones its CLI lacks: --greedy, --tokens, --n-predict, --ignore-eos, --seed, --device,
// --gpus N (tensor-parallel over devices D..D+N-1, one forked process each), --on-device, --prompt-batch N (prompt tokens
// per recorded step, 6..64 run on the tensor cores; default 1), --exact-prompt (batched prompt products with exact weight tiles), --write-synthetic, and --port / --bind for --server.
int llava_context::run(int argc, char** argv) {
    bool server_mode = false, only_print_header = false, greedy = false, ignore_eos = false, on_device = false;
    bool model_path_provided = false, have_seed = false, exact_prompt = false;
    string model_path, tokens_path, synth_spec, bind_address = "0.0.0.0";
    u32 server_port = 1337;
    string prompt = "The ten best monuments to see in Paris are";
    u32 n_predict = 0, seed = 0, gpus = 1, prompt_batch = 1;
    int device = 0;

    auto need_value = [&](int& i) -> const char* {
        if (i + 1 >= argc) {
            cerr << "[!] Expected a value after " << argv[i] << endl;
            exit(1);
        }
        return argv[++i];
    };
    for (int i = 1; i < argc; ++i) {
        const char* a = argv[i];
        if (streq(a, "--use-prebuilt") || streq(a, "--debug")) {
            // shader selection / Vulkan validation layer: nothing to select here
        } else if (streq(a, "--print_header")) {
            only_print_header = true;
        } else if (streq(a, "--model") || streq(a, "-m")) {
            if (model_path_provided) cerr << "[!] -m or --model duplicated in the command line" << endl;
            model_path_provided = true;
            model_path = need_value(i);
        } else if (streq(a, "--help") || streq(a, "-h")) {
            cout << (argc ? argv[0] : "./vulkan_llama")
                 << " [-h] [-m model.bin] [--server [--port P] [--bind ADDR]] [--greedy] [--n-predict N] [--ignore-eos] [--tokens ids.txt] [--seed S]"
                    " [--device D] [--gpus N] [--on-device] [--prompt-batch N] [--exact-prompt] [--print_header] [--write-synthetic 7b|13b|tiny[:q8][:layers=N]] [prompt]"
                 << endl;
            exit(0);
        } else if (streq(a, "--verbose") || streq(a, "-v")) {
            verbosity++;
        } else if (streq(a, "--control") || streq(a, "-c")) {
            cerr << "Control disabled for now" << endl;
            exit(1);
        } else if (streq(a, "--server") || streq(a, "-s")) {
            server_mode = true;
        } else if (streq(a, "--port")) {
            server_port = u32(strtoul(need_value(i), nullptr, 10));
        } else if (streq(a, "--bind")) {
            bind_address = need_value(i);
        } else if (streq(a, "--sigdebug")) {
            signal_debug = true;
        } else if (streq(a, "--greedy")) {
            greedy = true;
        } else if (streq(a, "--ignore-eos")) {
            ignore_eos = true;
        } else if (streq(a, "--on-device")) {
            on_device = true;
        } else if (streq(a, "--exact-prompt")) {
            exact_prompt = true;
        } else if (streq(a, "--prompt-batch")) {
            prompt_batch = u32(strtoul(need_value(i), nullptr, 10));
        } else if (streq(a, "--tokens")) {
            tokens_path = need_value(i);
        } else if (streq(a, "--n-predict")) {
            n_predict = u32(strtoul(need_value(i), nullptr, 10));
        } else if (streq(a, "--seed")) {
            seed = u32(strtoul(need_value(i), nullptr, 10));
            have_seed = true;
        } else if (streq(a, "--device")) {
            device = atoi(need_value(i));
        } else if (streq(a, "--gpus")) {
            gpus = u32(strtoul(need_value(i), nullptr, 10));
        } else if (streq(a, "--write-synthetic")) {
            synth_spec = need_value(i);
        } else if (i + 1 != argc) {
            cerr << "[!] Unexpected argument " << a << endl;
            exit(1);
        } else {
            prompt = a;
        }
    }

    if (model_path.empty()) {
        if (const char* env = ::getenv("LLAVA_MODEL")) model_path = env;      // llava_context.cpp:207-212
    }
    if (model_path.empty()) {
        cerr << "[!] No model path provided" << endl;
        exit(1);
    }

    if (!synth_spec.empty()) {
        synth_config cfg;
        stringstream ss(synth_spec);
        string part;
        bool first = true;
        while (getline(ss, part, ':')) {
            if (first) {
                first = false;
                if (part == "7b") { cfg.n_layers = 32; }
                else if (part == "13b") { cfg.dim = 5120; cfg.n_heads = 40; cfg.ff_size = 13824; cfg.n_layers = 40; }
                else if (part == "tiny") { cfg.n_layers = 2; }
                else { cerr << "[!] unknown synthetic model " << part << endl; return 1; }
            } else if (part == "q8") {
                cfg.wtype = ggml_value_type::q8_0;
            } else if (part.rfind("layers=", 0) == 0) {
                cfg.n_layers = u32(strtoul(part.c_str() + 7, nullptr, 10));
            } else if (part.rfind("seed=", 0) == 0) {
                cfg.seed = strtoull(part.c_str() + 5, nullptr, 10);
            }
        }
        string err;
        if (!synth_write_ggjt(model_path, cfg, &err)) {
            cerr << "[!] " << err << endl;
            return 1;
        }
        return 0;
    }

    if (only_print_header) {
        ggml_file f(model_path.c_str());
        if (!f.is_open()) return 1;
        f.print_info();
        return 0;
    }
    // --gpus N: the process forks N-1 times before anything touches CUDA; rank r drives device D + r, rank 0 (the
    // parent) speaks, the others run the same loop silently (same tokens: the ranks' logits are bit-identical)
    tp_rendezvous* rv = nullptr;
    u32 my_rank = 0;
    vector<pid_t> children;
    if (gpus == 0 || gpus > 8) {
        cerr << "[!] --gpus takes 1..8" << endl;
        return 1;
    }
    if (gpus > 1) {
        if (server_mode) {
            cerr << "[!] --server drives one GPU; --gpus is for the generation loop" << endl;
            return 1;
        }
        void* mem = ::mmap(nullptr, sizeof(tp_rendezvous), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
        if (mem == MAP_FAILED) {
            perror("mmap");
            return 1;
        }
        rv = new (mem) tp_rendezvous{};
        cout.flush();
        for (u32 r = 1; r < gpus; ++r) {
            const pid_t pid = ::fork();
            if (pid < 0) {
                perror("fork");
                rv->failed = 1;
                break;
            }
            if (pid == 0) {
                my_rank = r;
                children.clear();
                cout.setstate(ios::failbit);            // only rank 0 prints
                break;
            }
            children.push_back(pid);
        }
    }
    auto finish = [&](int code) -> int {
        if (rv == nullptr) return code;
        if (code != 0) rv->failed = 1;
        // no rank releases its peer window while another may still launch kernels that store into it: everyone
        // reports here once its own loop has ended (a rank that stopped early makes the others' bounded device waits
        // run out, which ends their loops too)
        rv->done.fetch_add(1, std::memory_order_acq_rel);
        const auto t0 = std::chrono::steady_clock::now();
        while (rv->done.load(std::memory_order_acquire) < gpus && std::chrono::steady_clock::now() - t0 < std::chrono::seconds(120))
            std::this_thread::sleep_for(std::chrono::milliseconds(1));
        if (my_rank != 0) ::_exit(code);
        for (pid_t pid : children) {
            int status = 0;
            if (::waitpid(pid, &status, 0) < 0 || !WIFEXITED(status) || WEXITSTATUS(status) != 0) code = code ? code : 1;
        }
        return code;
    };
    if (!setup_signal_handling()) {
        cerr << "[!] Cannot setup signal handling" << endl;
        return finish(1);
    }
    if (rv == nullptr) {
        if (!open(model_path, device)) return 1;
    } else {
        if (my_rank == 0) {
            if (lv_comm_unique_id(rv->nccl_id) != LV_OK) {
                cerr << "[!] cannot make a communicator id: " << lv_last_error_string() << endl;
                return finish(1);
            }
            rv->id_ready.store(1, std::memory_order_release);
        } else if (!rendezvous_wait(rv, rv->id_ready, 1)) {
            return finish(1);
        }
        if (!open_sharded(model_path, device + int(my_rank), my_rank, gpus, rv->nccl_id)) return finish(1);
        // peer windows for the exchange fused into the GEMVs: every rank publishes its handle, then maps the others'
        if (!peer_window_create(rv->handles[my_rank])) {
            cerr << "[!] rank " << my_rank << ": cannot create the peer window: " << lv_last_error_string() << endl;
            return finish(1);
        }
        rv->handles_ready.fetch_add(1, std::memory_order_acq_rel);
        if (!rendezvous_wait(rv, rv->handles_ready, gpus)) return finish(1);
        if (!peer_connect(&rv->handles[0][0])) {
            cerr << "[!] rank " << my_rank << ": cannot map the peers' windows: " << lv_last_error_string() << endl;
            return finish(1);
        }
        rv->connected.fetch_add(1, std::memory_order_acq_rel);
        if (!rendezvous_wait(rv, rv->connected, gpus)) return finish(1);
    }
    if (verbosity) cout << "Selected device: cuda:" << device << " (" << lv_ctx_sm_count(lv_context) << " SMs)" << endl;
    if (exact_prompt) lv_gemm_tc_set_exact(lv_context, 1);
    if (server_mode) {
        // llava_context.cpp:246-249: sessions are created and driven by the clients; standard input or a signal ends it
        lsrv::session_wrapper::set_deterministic_sessions(greedy);
        lsrv::session_wrapper::set_prompt_batch(prompt_batch);
        lsrv::tlv_server server(this, u16(server_port), bind_address.c_str(), true);
        if (!server.open()) return 1;
        server.serve_forever();
        return 0;
    }

    // generation loop, llava_context.cpp:336-373
    const u32 eos_id = 2;
    llava_session session(this);
    session.set_deterministic(greedy);
    if (have_seed) session.set_seed(seed);
    if (prompt_batch > 1 && !session.set_max_batch(prompt_batch)) {
        cerr << "[!] --prompt-batch takes 1.." << llava_session::max_batch_limit << " (sharded: 6 or more, where the shard shapes fit the tiles)" << endl;
        return finish(1);
    }
    if (!tokens_path.empty()) {
        vector<u32> ids;
        if (!read_token_file(tokens_path, &ids)) {
            cerr << "[!] cannot read token ids from " << tokens_path << endl;
            return finish(1);
        }
        for (u32 t : ids) {
            if (!session.push_token(t)) {
                cerr << "[!] System prompt overflows backlog buffer !" << endl;
                return finish(1);
            }
        }
    } else {
        if (!session.set_text(prompt)) {
            cerr << "[!] System prompt overflows backlog buffer !" << endl;
            return finish(1);
        }
        cout << prompt << flush;
    }

    u32 produced = 0;
    if (on_device && greedy && n_predict > 1) {
        // evaluate the prompt, then let the device feed itself
        u32 tok = session.predict_next_token();
        if (~tok == 0 || !session.push_token(tok)) return finish(1);
        vector<u32> rest;
        if (!session.generate_greedy_on_device(n_predict - 1, &rest)) {
            cerr << "Unknown error" << endl;
            return finish(1);
        }
        cout << model->get_tokens()[tok].text;
        for (u32 t : rest) cout << model->get_tokens()[t].text;
        cout << endl;
        return finish(0);
    }
    int status = 0;
    u32 next_token = session.predict_next_token();
    while (true) {
        if (~next_token == 0) {
            cerr << "Unknown error" << endl;
            status = 1;
            break;
        }
        ++produced;
        if (pop_signal() || (next_token == eos_id && !ignore_eos)) break;
        if (n_predict && produced >= n_predict) break;
        if (!session.push_token(next_token)) break;      // too many tokens
        if (!session.start_next_token_prediction()) {
            cerr << "Cannot start processing, unknown error" << endl;
            status = 1;
            break;
        }
        cout << model->get_tokens()[next_token].text << flush;     // printed while the device works
        next_token = session.finish_next_token_prediction();
    }
    if (~next_token != 0 && (next_token != eos_id || ignore_eos)) cout << model->get_tokens()[next_token].text;
    cout << endl;
    return finish(status);
}
