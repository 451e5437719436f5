"""Low-precision training: MX quantisers (`mx`), MXFP8 linear / grouped autograd (`mx_linear`), block-FP8 linear
(`block_fp8`), MXFP4 storage format (`mxfp4`), the `MXFP8Converter` (`mx_converter`), parameter-level quantisation
(`qat`) and its filters (`filters`)."""
