#include "pb_kern.h"
char *pb_classify_aot(PbKern *k, const char *fn_name) { (void)k; (void)fn_name; return NULL; }
