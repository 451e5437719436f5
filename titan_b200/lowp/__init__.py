"""Low-precision training: MX (microscaling) FP8 linears / grouped experts and parameter-level fake quantisation."""
