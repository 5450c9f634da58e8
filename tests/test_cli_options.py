"""The command line takes the reference's option names (python/logssms/server/args.py:60-251 for the engine,
examples/chat.py:323-334 for sampling) where the engine has the option at all."""
import pytest

from logssms_b200.cli import Chat, build_parser


def test_reference_option_names_parse():
    args = build_parser().parse_args([
        "--model", "/m", "--dtype", "float32", "--dummy-weight", "--max-running-requests", "7",
        "--max-seq-len-override", "4096", "--memory-ratio", "0.5", "--max-prefill-tokens", "512",
        "--scheduling-policy", "prefill-first", "--mixed-prefill-tokens", "128", "--num-pages", "33",
        "--page-size", "128", "--max-tokens", "9", "--temperature", "0.8", "--top-k", "40", "--top-p", "0.95",
        "--ignore-eos", "--system", "be brief"])
    assert args.model_path == "/m" and args.dtype == "float32" and args.dummy_weight
    assert (args.max_running_requests, args.max_seq_len_override, args.memory_ratio) == (7, 4096, 0.5)
    assert (args.max_prefill_tokens, args.scheduling_policy, args.mixed_prefill_tokens) == (512, "prefill-first", 128)
    assert (args.num_pages, args.page_size) == (33, 128)
    assert (args.max_tokens, args.temperature, args.top_k, args.top_p, args.ignore_eos) == (9, 0.8, 40, 0.95, True)
    assert args.system == "be brief" and not args.no_graph and args.profile is None and not args.nvtx
    assert args.cuda_graph_max_bs is None
    args = build_parser().parse_args(["--model", "/m", "--profile", "/tmp/p.json", "--nvtx", "--no-graph"])
    assert args.profile == "/tmp/p.json" and args.nvtx and args.no_graph
    # the reference's two spellings of the graph option (0: no graphs; a number: the largest decode batch with a graph)
    assert build_parser().parse_args(["--model", "/m", "--cuda-graph-max-bs", "16"]).cuda_graph_max_bs == 16
    assert build_parser().parse_args(["--model", "/m", "--graph", "0"]).cuda_graph_max_bs == 0
    # an option of this engine alone: the dtype in which recurrent states are kept between steps
    assert build_parser().parse_args(["--model", "/m"]).ssm_state_dtype == "float32"
    assert build_parser().parse_args(["--model", "/m", "--ssm-state-dtype", "activation"]).ssm_state_dtype == "activation"
    with pytest.raises(SystemExit):
        build_parser().parse_args(["--model", "/m", "--ssm-state-dtype", "float16"])


def test_model_path_has_both_spellings_and_defaults_follow_the_chat_client():
    args = build_parser().parse_args(["--model-path", "/m"])
    assert args.model_path == "/m"
    assert (args.temperature, args.top_k, args.top_p, args.max_tokens) == (0.7, -1, 1.0, 1024)
    assert args.scheduling_policy == "mixed" and args.mixed_prefill_tokens is None


def test_unknown_policy_and_dtype_are_refused():
    for bad in (["--scheduling-policy", "decode-first"], ["--dtype", "float16"]):
        with pytest.raises(SystemExit):
            build_parser().parse_args(["--model", "/m", *bad])


class FakeLLM:
    """Stands in for `LLM` under the chat loop: records the prompts and answers with their length."""

    def __init__(self, tokenizer=None, fail_on=None):
        self.tokenizer, self.fail_on, self.prompts = tokenizer, fail_on, []

    def generate(self, prompts, params):
        from logssms_b200.engine.llm import Output
        self.prompts.append(list(prompts[0]))
        if self.fail_on is not None and len(self.prompts) == self.fail_on:
            raise RuntimeError("out of pages")
        ids = [len(prompts[0]), 1]
        text = self.tokenizer.decode(ids) if self.tokenizer is not None else None
        return [Output(ids, "length", text, list(prompts[0]))]


class FakeTokenizer:
    """Words of the form t<number>; no chat template: the turns are joined by newlines."""
    chat_template = None

    def encode(self, text):
        return [int(w[1:]) for w in text.split() if w[0] == "t"]

    def decode(self, ids):
        return " ".join(f"t{i}" for i in ids)


def chat(lines, **kw):
    import io
    out = io.StringIO()
    llm = FakeLLM(**kw)
    c = Chat(llm, params=None, system=None, out=out)
    c.loop(iter(lines))
    return c, llm, out.getvalue().splitlines()


def test_chat_loop_runs_every_command_of_the_reference_client_on_token_ids():
    """examples/chat.py:120-124: /help /new /list /switch /rename /delete /clear /system /history /exit."""
    assert set(Chat.COMMANDS) == {"/help", "/new", "/list", "/switch", "/rename", "/delete", "/clear", "/system",
                                  "/history", "/exit"}
    c, llm, said = chat([
        "/help", "5 6 7", "8, 9", "/history", "/new work", "1 2", "/list", "/switch chat-1", "3", "/rename first",
        "/list", "/switch nowhere", "/delete work", "/delete first", "/clear", "/history", "4", "/system be brief",
        "/frobnicate", "not ids", "", "/exit", "99"])
    # the history of a conversation is fed back: second turn = first prompt + its answer + the new ids
    assert llm.prompts[0] == [5, 6, 7] and llm.prompts[1] == [5, 6, 7, 3, 1, 8, 9]
    assert llm.prompts[2] == [1, 2]                                  # a new conversation starts empty
    assert llm.prompts[3] == [5, 6, 7, 3, 1, 8, 9, 7, 1, 3]          # back in chat-1
    assert llm.prompts[4] == [4]                                     # after /clear
    assert len(llm.prompts) == 5                                     # nothing ran after /exit, nor for "not ids"
    assert said[0].startswith("commands:") and sum(line.lstrip().startswith("/") for line in said) >= 10
    assert "3 1   [length]" in said and "7 1   [length]" in said
    assert "[user] [5, 6, 7]" in said and "[assistant] [3, 1]" in said
    assert "now in work" in said and "* work (2 turns)" in said and "  chat-1 (4 turns)" in said
    assert "* first (6 turns)" in said                               # after /rename
    assert "no conversation 'nowhere'" in said
    assert "cannot delete that" in said                              # the last conversation stays
    assert any("unknown command /frobnicate" in line for line in said)
    assert any("type token ids" in line for line in said)
    assert said[-1] == "bye" and c.system == "be brief" and list(c.conversations) == ["first"]


def test_chat_loop_with_a_tokenizer_builds_the_prompt_from_system_and_turns_and_survives_an_error():
    c, llm, said = chat(["/system t1 t2", "t5 t6", "t7", "t8", "/history", "/exit"], tokenizer=FakeTokenizer(), fail_on=3)
    assert llm.prompts[0] == [1, 2, 5, 6]                            # system prompt, then the user's words
    assert llm.prompts[1] == [1, 2, 5, 6, 4, 1, 7]                   # ... the answer (t4 t1) and the next turn
    assert "t4 t1" in said and "t7 t1" in said
    assert any(line.startswith("Error: out of pages") for line in said)
    assert said.count("[user] t8") == 0                              # the failed turn left no history
    assert said[-1] == "bye"
