// bin/trace_run: feeds given token ids through the engine step by step and writes logits.
//     trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N < steps.jsonl
// The work is the library's own replay over its model, step function, cache and kernels.
#include "../../include/liyab_b200.h"

int main(int argc, char** argv) { return lb_trace_run_main(argc, argv); }
