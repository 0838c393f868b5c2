"""LlamaConversation (src/models/transformer/conversation.rs:29-85) behind include/rg_b200_workflow.h, driven
through a table of Python callables: the transcript is staged per turn and committed only on success."""
import pytest

from rustgrad_b200 import workflow


class FakeChat(workflow.ChatBackend):
    """Answers with the number of messages it was shown; can be told to fail once."""

    def __init__(self):
        self.seen, self.fail = [], None

    def generate_chat(self, messages, max_new_tokens):
        self.seen.append((list(messages), max_new_tokens))
        if self.fail:
            rc, tok = self.fail
            self.fail = None
            return rc, tok, 0, [], "", False
        text = f"reply {len(messages)}"
        generated = list(range(min(max_new_tokens, 3)))
        return 0, 0, 10 * len(messages), generated, text if generated else "", False


def test_turns_extend_the_transcript_and_failures_leave_it_alone():
    chat = FakeChat()
    conv = workflow.LlamaConversation(chat)
    assert conv.history() == [] and conv.cache_len() == 0
    turn = conv.send("hello", 8)
    assert turn.user == ("user", "hello") and turn.assistant == ("assistant", "reply 1")
    assert turn.generation.generated_ids == [0, 1, 2] and turn.generation.decoded == "reply 1"
    assert conv.history() == [("user", "hello"), ("assistant", "reply 1")]
    assert conv.cache_len() == 10 + 3 - 1  # the prompt and all but the last generated id
    # the next turn shows the model the whole staged transcript
    conv.send("and then?", 8)
    assert chat.seen[-1] == ([("user", "hello"), ("assistant", "reply 1"), ("user", "and then?")], 8)
    assert conv.history()[-1] == ("assistant", "reply 3") and conv.cache_len() == 30 + 3 - 1
    # empty input is refused before anything runs
    calls = len(chat.seen)
    with pytest.raises(workflow.ConversationError) as e:
        conv.send("", 8)
    assert e.value.kind == "EmptyInput" and len(chat.seen) == calls
    # a message over the bound is a chat error, checked before the empty-input rule can matter
    with pytest.raises(workflow.ConversationError) as e:
        conv.send("x" * (1024 * 1024 + 1), 8)
    assert (e.value.kind, e.value.detail) == ("Chat", 16) and len(chat.seen) == calls
    # a template / tokenizer failure and a generation failure: transcript and cache length stay
    before = (conv.history(), conv.cache_len())
    chat.fail = (2, 9)  # RG_INVALID_ARGUMENT with a tokenizer status
    with pytest.raises(workflow.ConversationError) as e:
        conv.send("breaks", 8)
    assert (e.value.kind, e.value.detail) == ("Chat", 9)
    chat.fail = (7, 0)  # a session status
    with pytest.raises(workflow.ConversationError) as e:
        conv.send("breaks too", 8)
    assert (e.value.kind, e.value.detail) == ("Generation", 7)
    assert (conv.history(), conv.cache_len()) == before
    # no new tokens: an empty assistant message is committed, the cache is left as it was
    conv.send("quiet", 0)
    assert conv.history()[-2:] == [("user", "quiet"), ("assistant", "")] and conv.cache_len() == before[1]
    conv.reset()
    assert conv.history() == [] and conv.cache_len() == 0
    assert conv.send("again", 2).assistant == ("assistant", "reply 1")
