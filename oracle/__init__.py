"""TEST INFRASTRUCTURE: CPU oracle for the causal-attention path (see oracle/attn_oracle.c)."""
