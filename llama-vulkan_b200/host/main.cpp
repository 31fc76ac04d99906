// vulkan_llama command-line tool (main.cpp:3-7 of the reference).
#include "llava_context.h"

int main(int argc, char** argv) {
    llava_context context;
    return context.run(argc, argv);
}
