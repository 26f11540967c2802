#include "velomind_b200/velomind.h"
int main(int argc, char** argv) { return vmb::trace_run_main(argc, argv); }
