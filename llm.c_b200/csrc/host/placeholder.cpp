extern "C" int llmc_host_version() { return 1; }
