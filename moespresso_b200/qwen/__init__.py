"""Qwen / Ornith full-attention prefill operator."""
