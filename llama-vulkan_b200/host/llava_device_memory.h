// Device arena: buffers register their size before freeze(), which makes the
// single allocation.  Counterpart of the reference's llava_device_memory
// (llava_device_memory.h:16-30) on top of lv_arena_create.
#ifndef LLAVA_B200_DEVICE_MEMORY_H
#define LLAVA_B200_DEVICE_MEMORY_H

#include <set>
#include <string>

#include "types.h"

class llava_device_memory {
public:
    explicit llava_device_memory(llava_context* context);
    ~llava_device_memory();
    llava_device_memory(const llava_device_memory&) = delete;
    llava_device_memory& operator=(const llava_device_memory&) = delete;

    bool is_frozen() const { return base != nullptr; }
    bool freeze();                                       // allocates; false on failure
    void register_llava_buffer(llava_buffer* buffer);
    void forget_llava_buffer(llava_buffer* buffer);
    size_t register_buffer(size_t alignment, size_t buffer_size);   // -> offset in the arena
    size_t get_size() const { return cursor; }
    u8* device_base() const { return base; }

    // Host <-> arena copies; they stand in for the reference's map()/unmap() of
    // host-visible Vulkan memory.  Blocking, ordered after work already enqueued.
    bool write(size_t offset, const void* src, size_t size) const;
    bool read(size_t offset, void* dst, size_t size) const;
    bool zero(size_t offset, size_t size) const;

    // Trace frames: every f32 buffer of the arena except the KV caches, sorted by name.
    void dump_buffers(int out_fd, const std::string& name);

    llava_context* const context;

private:
    u8* base = nullptr;
    size_t cursor = 0;
    std::set<llava_buffer*> buffers;
};

#endif
