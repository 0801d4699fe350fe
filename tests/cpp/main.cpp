// Runner of the native test layer: `ob_native_tests [substring-filter]`.
#include "check.h"

int main(int argc, char** argv) { return obtest::run_all(argc > 1 ? argv[1] : nullptr) == 0 ? 0 : 1; }
