"""Command line: `python -m logssms_b200 --model-path DIR [...]`.

An in-process stand-in for the reference's server + chat client pair: engine options carry the
names of the reference's server flags (python/logssms/server/args.py:60-251), the chat loop the
commands and sampling options of its chat client (examples/chat.py:120-124, 323-334).  Without a
tokenizer in the model folder (a random-weights model) prompts are typed as token ids.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile

HELP = """commands:
  /help               this text
  /new [name]         start a new conversation
  /list               list conversations
  /switch <name>      continue another conversation
  /rename <name>      rename the current conversation
  /delete <name>      delete a conversation
  /clear              forget the current conversation's history
  /system <text>      set the system prompt (tokenizer models only)
  /history            print the current conversation
  /exit               quit"""


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="python -m logssms_b200", description=__doc__,
                                formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model-path", "--model", required=True,
                   help="model folder (config.json + safetensors); with --dummy-weight only config.json is read")
    p.add_argument("--dtype", default="auto", choices=["auto", "bfloat16", "float32"])
    p.add_argument("--dummy-weight", action="store_true", help="seeded random weights instead of the checkpoint")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--max-running-requests", type=int, default=64)
    p.add_argument("--max-seq-len-override", type=int, default=None)
    p.add_argument("--max-prefill-tokens", type=int, default=8192, help="token budget of one step")
    p.add_argument("--scheduling-policy", default="mixed", choices=["mixed", "prefill-first"],
                   help="mixed: prompt portions beside decoded tokens in one step; prefill-first: prompts before decoding")
    p.add_argument("--mixed-prefill-tokens", type=int, default=None,
                   help="most prompt tokens in a step that also decodes (mixed policy; default: the step's budget)")
    p.add_argument("--no-graph", action="store_true", help="launch every step kernel by kernel (no CUDA graphs)")
    p.add_argument("--cuda-graph-max-bs", "--graph", type=int, default=None, dest="cuda_graph_max_bs",
                   help="largest decode batch that gets a CUDA graph; the batch sizes 1, 2, 4, 8, 16, ... up to it are "
                        "captured at start.  0 disables all graphs; default: every batch size, captured when it comes twice")
    p.add_argument("--ssm-state-dtype", choices=["float32", "activation"], default="float32",
                   help="dtype in which recurrent states are kept between steps: float32, or the model's dtype (as the "
                        "reference keeps them: half the bytes of a decode step's state update, one rounding per step)")
    p.add_argument("--profile", default=None, metavar="FILE",
                   help="time every kernel with CUDA events and write the sums per kernel class to FILE (JSON) at exit; "
                        "such a run launches every step kernel by kernel")
    p.add_argument("--nvtx", action="store_true", help="NVTX ranges per layer and part, for a timeline tool")
    p.add_argument("--memory-ratio", type=float, default=0.9)
    p.add_argument("--num-pages", type=int, default=None)
    p.add_argument("--page-size", type=int, default=64)
    # sampling, as the chat client names them
    p.add_argument("--max-tokens", type=int, default=1024)
    p.add_argument("--temperature", type=float, default=0.7)
    p.add_argument("--top-k", type=int, default=-1)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--system", default=None, help="initial system prompt")
    p.add_argument("--prompt-ids", default=None,
                   help="comma-separated token ids: generate once, print the new ids, exit")
    return p


def _model_folder(args) -> str:
    if not args.dummy_weight:
        return args.model_path
    import torch
    from .config import load_model_config
    from .weights import write_random_model
    out = tempfile.mkdtemp(prefix="logssms_b200_dummy_")
    dtype = torch.float32 if args.dtype == "float32" else torch.bfloat16
    write_random_model(load_model_config(args.model_path), out, seed=args.seed, dtype=dtype)
    for name in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json", "special_tokens_map.json"):
        src = os.path.join(args.model_path, name)
        if os.path.isfile(src):
            os.symlink(os.path.abspath(src), os.path.join(out, name))
    return out


class Chat:
    COMMANDS = ("/help", "/new", "/list", "/switch", "/rename", "/delete", "/clear", "/system", "/history", "/exit")

    def __init__(self, llm, params, system=None, out=sys.stdout):
        self.llm, self.params, self.out = llm, params, out
        self.system = system
        self.conversations: dict[str, list] = {"chat-1": []}
        self.current = "chat-1"

    def say(self, text: str) -> None:
        print(text, file=self.out, flush=True)

    def command(self, line: str) -> bool:
        """Run a slash command; False means quit."""
        cmd, _, arg = line.partition(" ")
        arg = arg.strip()
        if cmd == "/exit":
            return False
        if cmd == "/help":
            self.say(HELP)
        elif cmd == "/new":
            name = arg or f"chat-{len(self.conversations) + 1}"
            self.conversations.setdefault(name, [])
            self.current = name
            self.say(f"now in {name}")
        elif cmd == "/list":
            for name, turns in self.conversations.items():
                self.say(f"{'*' if name == self.current else ' '} {name} ({len(turns)} turns)")
        elif cmd == "/switch":
            if arg in self.conversations:
                self.current = arg
            else:
                self.say(f"no conversation {arg!r}")
        elif cmd == "/rename":
            if arg and arg not in self.conversations:
                self.conversations[arg] = self.conversations.pop(self.current)
                self.current = arg
            else:
                self.say("give a new, unused name")
        elif cmd == "/delete":
            if arg in self.conversations and len(self.conversations) > 1:
                del self.conversations[arg]
                if self.current == arg:
                    self.current = next(iter(self.conversations))
            else:
                self.say("cannot delete that")
        elif cmd == "/clear":
            self.conversations[self.current] = []
        elif cmd == "/system":
            self.system = arg or None
        elif cmd == "/history":
            for role, content in self.conversations[self.current]:
                self.say(f"[{role}] {content}")
        else:
            self.say(f"unknown command {cmd}; /help lists them")
        return True

    def turn(self, line: str) -> None:
        turns = self.conversations[self.current]
        tok = self.llm.tokenizer
        if tok is None:
            try:
                new_ids = [int(t) for t in line.replace(",", " ").split()]
            except ValueError:
                self.say("this model has no tokenizer: type token ids, e.g. 12 7 301")
                return
            ids = [t for role, content in turns for t in content] + new_ids
            out = self.llm.generate([ids], self.params)[0]
            turns += [("user", new_ids), ("assistant", out.token_ids)]
            self.say(" ".join(map(str, out.token_ids)) + f"   [{out.finish_reason}]")
            return
        messages = ([{"role": "system", "content": self.system}] if self.system else [])
        messages += [{"role": r, "content": c} for r, c in turns] + [{"role": "user", "content": line}]
        if getattr(tok, "chat_template", None):
            ids = tok.apply_chat_template(messages, add_generation_prompt=True, tokenize=True)
        else:
            ids = tok.encode("\n".join(m["content"] for m in messages))
        out = self.llm.generate([list(ids)], self.params)[0]
        turns += [("user", line), ("assistant", out.text)]
        self.say(out.text)

    def loop(self, lines) -> None:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            if line.startswith("/"):
                if not self.command(line):
                    break
            else:
                try:
                    self.turn(line)
                except (RuntimeError, ValueError) as exc:
                    self.say(f"Error: {exc}")
        self.say("bye")


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from .engine import LLM
    from .sampling import SamplingParams
    llm = LLM(_model_folder(args), args.dtype, max_running_requests=args.max_running_requests,
              max_seq_len_override=args.max_seq_len_override, page_size=args.page_size, num_pages=args.num_pages,
              memory_ratio=args.memory_ratio, max_prefill_tokens=args.max_prefill_tokens, seed=args.seed,
              scheduling_policy=args.scheduling_policy, mixed_prefill_tokens=args.mixed_prefill_tokens,
              use_graphs=not args.no_graph, profile=args.profile is not None, nvtx=args.nvtx,
              cuda_graph_max_bs=args.cuda_graph_max_bs, ssm_state_dtype=args.ssm_state_dtype)
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            ignore_eos=args.ignore_eos, max_tokens=args.max_tokens)
    def write_profile():
        if args.profile is not None:
            import json
            with open(args.profile, "w") as f:
                json.dump(llm.engine.profile_report(), f, indent=1)

    if args.prompt_ids is not None:
        ids = [int(t) for t in args.prompt_ids.replace(",", " ").split()]
        out = llm.generate([ids], params)[0]
        print(" ".join(map(str, out.token_ids)))
        write_profile()
        return 0
    chat = Chat(llm, params, args.system)
    print("logssms_b200 chat; /help for commands", flush=True)

    def lines():
        while True:
            try:
                yield input(f"{chat.current}> ")
            except EOFError:
                return
            except KeyboardInterrupt:
                print("\nCancelled. Use /exit or Ctrl-D to quit.")
    chat.loop(lines())
    write_profile()
    return 0
