"""
Interactive chat with a checkpoint (``python -m olmo_core_b200.generate.chat CHECKPOINT_DIR``; role of
src/olmo_core/generate/chat.py:47-462).

The conversation is a list of ``{"role", "content"}`` messages rendered to a prompt with a Jinja chat template (by
default the messages are simply concatenated), generated from with :class:`TransformerGenerationModule` and appended to.
``/clear`` drops the history (keeping the system prompt), ``/help`` lists the commands, ``/quit`` or ``/exit`` leaves.
:class:`ChatSession` holds that logic without any terminal I/O, so it can be scripted and tested; :func:`main` is the
terminal front end (colour through ``rich`` when it is installed).
"""

from __future__ import annotations

import argparse
import json
import logging
import sys
from typing import Any, Callable, Dict, List, Optional

import torch

from ..aliases import PathOrStr
from ..config import DType
from ..data import TokenizerConfig
from ..io import join_path, normalize_path, read_text
from ..nn.attention import AttentionBackendName
from ..utils import get_default_device, prepare_cli_environment
from .generation_module import GenerationConfig, TransformerGenerationModule

log = logging.getLogger(__name__)

__all__ = ["DEFAULT_CHAT_TEMPLATE", "ChatSession", "load_tokenizer", "load_tokenizer_config_from_checkpoint", "main"]

DEFAULT_CHAT_TEMPLATE = "{% for message in messages %}{{ message['content'] }}{% endfor %}"
HELP_TEXT = ("Commands:\n  /quit or /exit - Exit the chatbot\n  /clear - Clear conversation history\n"
             "  /help - Show this help message")


def load_tokenizer(tokenizer_config: TokenizerConfig):
    """The Hugging Face tokenizer named by the config's identifier."""
    if tokenizer_config.identifier is None:
        raise ValueError("Tokenizer config has no identifier. Cannot load tokenizer.")
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(tokenizer_config.identifier)


def load_tokenizer_config_from_checkpoint(checkpoint_dir: PathOrStr) -> Optional[TokenizerConfig]:
    """From ``<checkpoint>/config.json`` (written by the config-saver callback); ``None`` if it is not there."""
    path = join_path(normalize_path(checkpoint_dir), "config.json")
    try:
        return TokenizerConfig.from_dict(json.loads(read_text(path))["dataset"]["tokenizer"])
    except (KeyError, FileNotFoundError, OSError) as e:
        log.warning("Could not load tokenizer config from checkpoint: %s", e)
        return None


class ChatSession:
    """Conversation state + one ``respond`` step; I/O free."""

    def __init__(self, generation_module: Any, tokenizer: Any, *, system_prompt: Optional[str] = None,
                 chat_template: str = DEFAULT_CHAT_TEMPLATE, show_special_tokens: bool = False):
        self.module, self.tokenizer = generation_module, tokenizer
        self.system_prompt, self.chat_template = system_prompt, chat_template
        self.show_special_tokens = show_special_tokens
        self.history: List[Dict[str, str]] = []
        self.clear()

    def clear(self) -> None:
        self.history = [{"role": "system", "content": self.system_prompt}] if self.system_prompt else []

    def build_prompt(self) -> str:
        return self.tokenizer.apply_chat_template(self.history, tokenize=False, add_generation_prompt=True,
                                                  chat_template=self.chat_template)

    def respond(self, user_message: str) -> str:
        """Append the user message, generate, append and return the reply. On failure the user message is dropped again."""
        self.history.append({"role": "user", "content": user_message})
        try:
            input_ids = self.tokenizer.encode(self.build_prompt(), return_tensors="pt")
            generated, _, _ = self.module.generate_batch(input_ids, completions_only=True, log_timing=False)
            reply = self.tokenizer.decode(generated[0], skip_special_tokens=not self.show_special_tokens)
        except Exception:
            self.history.pop()
            raise
        self.history.append({"role": "assistant", "content": reply})
        return reply

    def handle(self, line: str) -> Optional[str]:
        """One line of user input → text to show (``None`` means: leave)."""
        line = line.strip()
        if not line:
            return ""
        command = line.lower()
        if command in ("/quit", "/exit"):
            return None
        if command == "/clear":
            self.clear()
            return "Conversation history cleared."
        if command == "/help":
            return HELP_TEXT
        return self.respond(line)


def _parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(
        description="Chat with a checkpoint through TransformerGenerationModule",
        formatter_class=argparse.RawDescriptionHelpFormatter,
        epilog=("Examples:\n  python -m olmo_core_b200.generate.chat /path/to/checkpoint\n"
                "  python -m olmo_core_b200.generate.chat /path/to/checkpoint --max-new-tokens 512 --temperature 0.7\n"
                "  python -m olmo_core_b200.generate.chat /path/to/checkpoint --no-do-sample"))
    p.add_argument("checkpoint_dir", type=str, help="Path to checkpoint directory")
    p.add_argument("--max-new-tokens", type=int, default=1024)
    p.add_argument("--max-length", type=int, default=None, help="Prompt + generation; overrides --max-new-tokens.")
    p.add_argument("--temperature", type=float, default=1.0, help="0.0 means greedy decoding.")
    p.add_argument("--top-k", type=int, default=-1, help="-1 disables top-k filtering.")
    p.add_argument("--top-p", type=float, default=0.7)
    p.add_argument("--do-sample", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--use-cache", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--attention-backend", type=str, default=None, choices=[b.value for b in AttentionBackendName])
    p.add_argument("--dtype", type=str, default="bfloat16", choices=[d.value for d in DType])
    p.add_argument("--system-prompt", type=str, default=None)
    p.add_argument("--show-special-tokens", action="store_true")
    p.add_argument("--chat-template", type=str, default=DEFAULT_CHAT_TEMPLATE, help="Jinja2 chat template string.")
    p.add_argument("--verbosity", type=str, default="WARNING", choices=["DEBUG", "INFO", "WARNING", "ERROR", "CRITICAL"])
    return p


def _printer() -> Callable[[str, str], None]:
    try:
        from rich.console import Console
        from rich.panel import Panel

        console = Console()
        return lambda title, text: console.print(Panel(text, title=title, title_align="left"))
    except ImportError:
        return lambda title, text: print(f"[{title}]\n{text}\n")


def main(argv: Optional[List[str]] = None) -> None:
    args = _parser().parse_args(argv)
    logging.getLogger().setLevel(args.verbosity)
    show = _printer()
    tokenizer_config = load_tokenizer_config_from_checkpoint(args.checkpoint_dir) or TokenizerConfig.dolma2()
    tokenizer = load_tokenizer(tokenizer_config)
    show("Tokenizer", f"{tokenizer_config.identifier}: vocab {tokenizer_config.vocab_size}, "
                      f"eos {tokenizer_config.eos_token_id}, pad {tokenizer_config.pad_token_id}")
    generation_config = GenerationConfig(
        pad_token_id=tokenizer_config.pad_token_id, eos_token_id=tokenizer_config.eos_token_id,
        max_new_tokens=args.max_new_tokens if args.max_length is None else None, max_length=args.max_length,
        do_sample=args.do_sample, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
        use_cache=args.use_cache)
    try:
        module = TransformerGenerationModule.from_checkpoint(
            checkpoint_dir=args.checkpoint_dir, generation_config=generation_config, device=get_default_device(),
            dtype=DType(args.dtype),
            attention_backend=AttentionBackendName(args.attention_backend) if args.attention_backend else None)
    except Exception as e:
        log.error("Failed to load checkpoint: %s", e, exc_info=True)
        sys.exit(1)
    show("Generation config", str(generation_config))
    show("Welcome", "Chatbot ready! Type your message and press Enter.\n\n" + HELP_TEXT)
    session = ChatSession(module, tokenizer, system_prompt=args.system_prompt, chat_template=args.chat_template,
                          show_special_tokens=args.show_special_tokens)
    if args.system_prompt:
        show("System", args.system_prompt)
    while True:
        try:
            line = input("\nYou> ")
        except (EOFError, KeyboardInterrupt):
            print("\nGoodbye!")
            return
        try:
            with torch.inference_mode():
                reply = session.handle(line)
        except Exception as e:
            show("Error", str(e))
            continue
        if reply is None:
            print("Goodbye!")
            return
        if reply:
            show("Assistant" if not line.strip().startswith("/") else "Info", reply)


if __name__ == "__main__":
    prepare_cli_environment()
    main()


# ---------------------------------------------------------------------------------------------------------------
# Panels of the terminal front end (names of src/olmo_core/generate/chat.py:34-160; they need ``rich``)
# ---------------------------------------------------------------------------------------------------------------

def _bubble(message: str, title: str, colour: str, style: str):
    from rich.panel import Panel
    from rich.text import Text

    return Panel(Text(message, style=style), title=f"[bold {colour}]{title}[/bold {colour}]", title_align="left",
                 border_style=colour, padding=(0, 1))


def render_user_message(message: str):
    """A user turn as a chat bubble."""
    return _bubble(message, "User", "cyan", "default")


def render_assistant_message(message: str):
    """A model turn as a chat bubble."""
    return _bubble(message, "Assistant", "magenta", "default")


def render_system_message(message: str):
    """The system prompt, dimmed."""
    return _bubble(message, "System", "yellow", "dim")


def _two_columns(title: str, left: List[str], right: List[str], colour: str):
    from rich.columns import Columns
    from rich.panel import Panel
    from rich.text import Text

    return Panel(Columns([Text("\n".join(left)), Text("\n".join(right))], equal=True, expand=True),
                 title=f"[bold {colour}]{title}[/bold {colour}]", title_align="left", border_style=colour, padding=(0, 1))


def render_tokenizer_info(tokenizer_config: TokenizerConfig, tokenizer, chat_template: str):
    """The tokenizer settings of the checkpoint next to those of the loaded Hugging Face tokenizer."""
    left = ["OLMo-core TokenizerConfig:", f"  • Identifier: {tokenizer_config.identifier or 'N/A'}",
            f"  • Vocab size: {tokenizer_config.vocab_size:,}", f"  • EOS token ID: {tokenizer_config.eos_token_id}",
            f"  • Pad token ID: {tokenizer_config.pad_token_id}", f"  • BOS token ID: {tokenizer_config.bos_token_id}"]
    right = ["HuggingFace Tokenizer:", f"  • Vocab size: {getattr(tokenizer, 'vocab_size', 0):,}",
             f"  • Model max length: {getattr(tokenizer, 'model_max_length', None)}"]
    special = getattr(tokenizer, "all_special_tokens", None)
    if special:
        shown = ", ".join(special[:6]) + (", ..." if len(special) > 6 else "")
        right.append(f"  • Special tokens: {shown}")
    first_line = (chat_template or "").strip().splitlines()[0] if (chat_template or "").strip() else "N/A"
    right.append(f"  • Chat template: {first_line[:60]}")
    return _two_columns("Tokenizer", left, right, "green")


def render_generation_config(generation_config: GenerationConfig):
    """Sampling and cache settings of the session."""
    left = [f"• Max new tokens: {generation_config.max_new_tokens}"]
    right = [f"• Max length: {generation_config.max_length}"]
    if generation_config.do_sample:
        top_k = "unlimited" if generation_config.top_k == -1 else str(generation_config.top_k)
        left += ["• Sampling: enabled", f"• Temperature: {generation_config.temperature}", f"• Top-k: {top_k}",
                 f"• Top-p: {generation_config.top_p}"]
    else:
        left.append("• Sampling: disabled (greedy)")
    right.append(f"• KV cache: {'enabled' if generation_config.use_cache else 'disabled'}")
    return _two_columns("Generation config", left, right, "blue")
