"""B200-native mixed-bit codebook-quantized MoE expert layer (drop-in for DartMoQ-Qwen3.5)."""
