"""Safetensors helpers: layout probes and the multi-process Hugging Face → framework conversion."""
from .convert_safetensors import convert_hf_safetensors_multiprocess
from .utils import contains_safetensors_files, is_hf_safetensors_dir

__all__ = ["contains_safetensors_files", "convert_hf_safetensors_multiprocess", "is_hf_safetensors_dir"]
