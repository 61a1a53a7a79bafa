"""Python wrappers with the names, arguments and error behaviour of the reference's kernel
wrappers (reference: kernels/automatic_gefen_fused.py, automatic_vmean.py, exact_histogram_fused.py,
period_variance.py, lloyd_max_fused.py), calling the C ABI of libgefen_b200.so."""
