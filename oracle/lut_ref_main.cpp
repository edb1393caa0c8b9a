// Test infrastructure: command-line driver around the reference's header-only LUT class
// (kernels/csrc/kairos_kernel/lut/lut.h of the reference tree, included at build time from
// where it lies; no reference source is copied here).
//   lut_ref <n_records> (r id)*n  m m m ...   -> prints get(m) for every m, in order
#include <cstdio>
#include <cstdlib>

#include "lut.h"

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    LUT table;
    int i = 1;
    const int n = atoi(argv[i++]);
    for (int r = 0; r < n && i + 1 < argc; ++r) {
        const int right = atoi(argv[i++]);
        const int id = atoi(argv[i++]);
        table.record(right, id);
    }
    for (; i < argc; ++i) printf("%d ", table.get(atoi(argv[i])));
    printf("\n");
    return 0;
}
