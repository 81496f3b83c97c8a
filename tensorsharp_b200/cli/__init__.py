"""Command-line front end: one-shot inference, interactive chat, JSONL batch, benchmarks, diagnostics.

Parity: TensorSharp.Cli/Program.cs and InteractiveSession.cs.
"""
from .args import CliOptions, parse_cli_args, USAGE

__all__ = ["CliOptions", "parse_cli_args", "USAGE"]
