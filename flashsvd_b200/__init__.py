"""flashsvd_b200: B200 (sm_100a) decode path for SVD-factored Llama-shaped transformers."""
__version__ = "0.1.0"
