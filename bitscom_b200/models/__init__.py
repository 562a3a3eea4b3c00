"""Model families used by the trainers: Llama, GPT-2, ResNet."""
