// Host runtime library entry: version probe.
extern "C" int ds41_core_version() { return 1; }
