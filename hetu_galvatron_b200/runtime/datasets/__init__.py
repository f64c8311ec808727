"""Indexed token datasets (``.bin`` / ``.idx``), GPT sample packing with cached indices, dataset blending."""
