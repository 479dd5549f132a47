// Empty stand-in: the reference includes this header but uses nothing from it (see THC.h beside it).
