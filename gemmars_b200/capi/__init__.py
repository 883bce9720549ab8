"""The C API (include/gemmars_b200.h): ``build`` compiles it, ``host`` is what it calls."""
