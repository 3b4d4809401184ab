#include "../runtime/pb_runtime.h"
PbAotProgram *pb_make_gather(const PbHeader &, std::string &err) { err = "gather kernels not built"; return nullptr; }
PbAotProgram *pb_make_gemm(const PbHeader &, std::string &err) { err = "gemm kernels not built"; return nullptr; }
PbAotProgram *pb_make_copy(const PbHeader &, std::string &err) { err = "copy kernels not built"; return nullptr; }
