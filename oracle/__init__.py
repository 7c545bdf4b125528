"""CPU checker for the paged-attention path (test infrastructure, never shipped
on the product path).  See ``paged_attention_oracle`` for the functions."""
