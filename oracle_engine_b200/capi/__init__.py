"""The C API: `oe.h`, `liboe.so` (built by `build.py` from `oe_capi.cpp`) and the functions it calls (`bridge.py`)."""
