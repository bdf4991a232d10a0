"""Command lines in the manner of the reference's tools (positional arguments, same names and
defaults): ``python -m lightllm_b200.cli.<tool>``."""
