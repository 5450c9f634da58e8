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
    assert args.system == "be brief" and not args.no_graph


def test_model_path_has_both_spellings_and_defaults_follow_the_chat_client():
    args = build_parser().parse_args(["--model-path", "/m"])
    assert args.model_path == "/m"
    assert (args.temperature, args.top_k, args.top_p, args.max_tokens) == (0.7, -1, 1.0, 1024)
    assert args.scheduling_policy == "mixed" and args.mixed_prefill_tokens is None


def test_unknown_policy_and_dtype_are_refused():
    for bad in (["--scheduling-policy", "decode-first"], ["--dtype", "float16"]):
        with pytest.raises(SystemExit):
            build_parser().parse_args(["--model", "/m", *bad])


def test_chat_commands_are_the_reference_clients():
    assert set(Chat.COMMANDS) == {"/help", "/new", "/list", "/switch", "/rename", "/delete", "/clear", "/system",
                                  "/history", "/exit"}
