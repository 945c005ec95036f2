"""The entry point's tokenizers: a folder's own tokenizer (written here, a handful of words)
is found and used with its chat template; a folder without one gets bytes."""

import json

import pytest

from socrates_b200.engine.tokenizer import ByteTokenizer, encode_prompt, has_tokenizer_files, load_tokenizer

WORDS = {"<eos>": 0, "<unk>": 1, "hello": 2, "world": 3, "how": 4, "are": 5, "you": 6, "<assistant>": 7}
TEMPLATE = ("{% for m in messages %}{{ m['content'] }}{% endfor %}"
            "{% if add_generation_prompt %} <assistant>{% endif %}")


def write_tokenizer(folder, template=TEMPLATE):
    tokenizers = pytest.importorskip("tokenizers")
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel(WORDS, unk_token="<unk>"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.WhitespaceSplit()
    tok.save(str(folder / "tokenizer.json"))
    cfg = {"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<eos>", "unk_token": "<unk>"}
    if template is not None:
        cfg["chat_template"] = template
    (folder / "tokenizer_config.json").write_text(json.dumps(cfg))


def test_folder_tokenizer_is_found_and_used(tmp_path, monkeypatch):
    monkeypatch.setenv("HF_HUB_OFFLINE", "1")
    assert not has_tokenizer_files(tmp_path)
    assert isinstance(load_tokenizer(tmp_path, 256), ByteTokenizer)
    write_tokenizer(tmp_path)
    tok = load_tokenizer(tmp_path, 256)
    assert not isinstance(tok, ByteTokenizer)
    assert 0 in tok.all_special_ids                        # the stop set of the engine
    assert encode_prompt(tok, "hello world") == [2, 3, 7]  # template appended the generation prompt
    assert tok.decode([4, 5, 6]) == "how are you"
    with pytest.raises(ValueError):
        load_tokenizer(tmp_path, 4)                        # more ids than the model has


def test_folder_tokenizer_without_template(tmp_path, monkeypatch):
    monkeypatch.setenv("HF_HUB_OFFLINE", "1")
    write_tokenizer(tmp_path, template=None)
    tok = load_tokenizer(tmp_path, 256)
    assert encode_prompt(tok, "how are you") == [4, 5, 6]


def test_byte_tokenizer():
    wide = ByteTokenizer(300)
    ids = encode_prompt(wide, "héllo")
    assert ids == [b + 1 for b in "héllo".encode()] and 0 not in ids
    assert wide.decode(ids) == "héllo" and wide.decode([105, 299, 106]) == "h<299>i"
    small = ByteTokenizer(100)
    ids = encode_prompt(small, "hello")
    assert all(1 <= i < 100 for i in ids) and small.decode(ids) == " ".join(map(str, ids))
    assert encode_prompt(wide, "") != []                   # a prompt has at least one token
    with pytest.raises(ValueError):
        ByteTokenizer(1)
