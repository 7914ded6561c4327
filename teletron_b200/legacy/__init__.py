"""Drop-in modules with the reference's extension names (``fused_adaln``, ``fused_rmsnorm``)."""
