"""`lf.data`: DataLoader, Tokenizer, TextDataset (lua/luatorch/init.lua:21-25)."""
from .dataloader import DataLoader
from .dataset import TextDataset
from .tokenizer import Tokenizer

__all__ = ["DataLoader", "Tokenizer", "TextDataset"]
