"""Reference arm of the benchmark: the unmodified reference package (installed under
``baseline/_ref``) driving a stock-PyTorch model. Nothing here imports ``zenyx_b200``."""
