"""Model families: the HunyuanVideo-style MMDiT, the 3-D causal VAE and the text encoders."""
