"""End-to-end trainers: Llama DP x PP, GPT-2 sharded, ResNet-18 DDP."""
