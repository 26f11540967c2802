#include "velomind_b200/velomind.h"
int main(int argc, char** argv) { return vmb::smollm2_chat_main(argc, argv); }
