""""Dead to Rights": a terminal interrogation game that shows off guided decoding through the chat API.

    python -m deliverance_b200.agents.interrogation_game --url http://127.0.0.1:8080 [--seed 7] [--max-tokens 700]

Set-up uses three kinds of constrained generation (reference: nanocode-deliverance/.../game/DeadToRightsGame.java:101-250,
schemas :340-420): the suspect's name comes from a ``guided_regex`` with a hot temperature and a uniform pick inside the nucleus
(``uniform_top_p``), ten places and ten stolen items come from ``guided_json`` list schemas (one of each is drawn locally),
and the case file (public opening + hidden truth) is one ``guided_json`` object. Then the player questions the model, which
plays the guilty suspect; a good theory makes it confess with the marker ``<confession>true</confession>``.
Commands: ``/case`` (the public opening again), ``/reveal`` (the hidden truth), ``/quit``. Old turns are dropped from the
conversation beyond the case context and the most recent exchanges.
"""
from __future__ import annotations

import argparse
import json
import random
import re
import sys
from typing import Callable, Optional

SUSPECT_NAME_REGEX = "[A-Z][a-z]{2,12}( [A-Z][a-z]{2,12})?"
MARKER = "<confession>true</confession>"
CASE_CONTEXT_MESSAGES = 3   # system prompt, case file, public opening
RECENT_MESSAGES = 12


def choices_schema(field: str, n: int = 10) -> dict:
    return {"type": "object", "properties": {field: {"type": "array", "minItems": n, "maxItems": n, "items": {"type": "string", "maxLength": 40}}},
            "required": [field], "additionalProperties": False}


def case_file_schema() -> dict:
    text = {"type": "string", "maxLength": 160}
    return {"type": "object", "additionalProperties": False,
            "properties": {"case_title": {"type": "string", "maxLength": 60}, "setting": text,
                           "clues": {"type": "array", "minItems": 3, "maxItems": 3, "items": text},
                           "hidden": {"type": "object", "additionalProperties": False,
                                      "properties": {"what_happened": text, "motive": text, "method": text, "mistake": text},
                                      "required": ["what_happened", "motive", "method", "mistake"]}},
            "required": ["case_title", "setting", "clues", "hidden"]}


def system_prompt() -> str:
    return ("You are running a fictional interrogation mystery game called Dead to Rights. You are the guilty suspect being questioned by "
            "the user; the crime is non-violent (a theft). Answer every question in first person. Pretend to be innocent but keep the "
            "mystery fun: give specific details, partial truths and suspicious excuses the user can follow up on, consistent with the hidden "
            "truth of the case file. If the user presents a theory that connects you to the crime through the clues or your contradictions, "
            f"break down, admit what you did and why, and only then include exactly this marker: {MARKER}")


def confessed(text: Optional[str]) -> bool:
    return bool(text) and MARKER in text.lower()


def clean_choice(text: str) -> str:
    return re.sub(r"^[\s,;:.\-]+", "", (text or "").replace("_", " ")).strip()


def trim_conversation(messages: list) -> None:
    keep = CASE_CONTEXT_MESSAGES + RECENT_MESSAGES
    if len(messages) > keep:
        messages[:] = messages[:CASE_CONTEXT_MESSAGES] + messages[-RECENT_MESSAGES:]


class Game:
    """``chat(messages, **request_fields) -> reply text``; ``ask() -> next input line or None``; ``say(text)`` prints."""

    def __init__(self, chat: Callable[..., str], ask: Callable[[], Optional[str]], say: Callable[[str], None], seed: int = 0,
                 temperature: float = 0.7, max_tokens: int = 700):
        self.chat, self.ask, self.say = chat, ask, say
        self.rng = random.Random(seed)
        self.temperature, self.max_tokens = temperature, max_tokens
        self.case: dict = {}
        self.messages: list = []

    def _json(self, system: str, user: str, schema: dict, temperature: float) -> dict:
        reply = self.chat([{"role": "system", "content": system}, {"role": "user", "content": user + " Return only JSON matching the schema."}],
                          guided_json=schema, temperature=temperature, max_tokens=self.max_tokens)
        try:
            return json.loads(reply)
        except ValueError as e:
            raise RuntimeError(f"the reply is not complete JSON (raise --max-tokens?): {reply[-80:]!r}") from e

    def setup(self) -> dict:
        name = self.chat([{"role": "system", "content": "You create concise ordinary fictional names for a light mystery game."},
                          {"role": "user", "content": "Generate only one fictional suspect name. No title, no explanation."}],
                         guided_regex=SUSPECT_NAME_REGEX, temperature=1.3, top_p=0.95, uniform_top_p=1.0, max_tokens=32).replace('"', "").strip()
        self.say(f"The suspect's name is {name}")
        picks = {}
        for field, what in (("places", "ordinary present-day locations (a bakery, a radio station, a bookshop, a museum office ...)"),
                            ("items", "ordinary objects that could be stolen (a trophy, a ledger, a signed book, a cash box ...)")):
            got = self._json("You generate varied setup options for a light, non-violent mystery game.", f"Generate 10 {what}.", choices_schema(field), 1.2)
            values = [clean_choice(v) for v in got.get(field, []) if isinstance(v, str) and v.strip()]
            if len(values) < 10:
                raise RuntimeError(f"expected 10 {field}, got {values}")
            picks[field] = self.rng.choice(values[:10])
            self.say(f"{field}: " + "; ".join(values[:10]) + f"\nselected: {picks[field]}")
        case = self._json(system_prompt(), f"Create the case file. The suspect is {name}; the place is {picks['places']}; the stolen item is "
                          f"{picks['items']}. Write three clues that point toward the suspect and the hidden truth.", case_file_schema(), self.temperature)
        case["suspect"] = name
        self.case = case
        self.messages = [{"role": "system", "content": system_prompt()},
                         {"role": "user", "content": "Case file (keep the hidden part secret until you confess): " + json.dumps(case)},
                         {"role": "assistant", "content": self.public_opening()}]
        self.say(self.public_opening())
        return case

    def public_opening(self) -> str:
        c = self.case
        return f"CASE: {c['case_title']}\nSUSPECT: {c['suspect']}\nSETTING: {c['setting']}\nCLUES:\n" + "\n".join(f"  {i + 1}. {x}" for i, x in enumerate(c["clues"]))

    def hidden_truth(self) -> str:
        return "\n".join(f"{k.replace('_', ' ')}: {v}" for k, v in self.case["hidden"].items())

    def play(self) -> str:
        """Runs until a confession ("confessed"), /quit or end of input ("closed")."""
        if not self.case:
            self.setup()
        while True:
            line = self.ask()
            if line is None or line.strip().lower() in ("/quit", "/q"):
                self.say("case closed")
                return "closed"
            line = line.strip()
            if not line:
                continue
            if line.lower() == "/reveal":
                self.say("HIDDEN TRUTH\n" + self.hidden_truth())
                continue
            if line.lower() == "/case":
                self.say(self.public_opening())
                continue
            self.messages.append({"role": "user", "content": f"Interrogator asks: {line}\nAnswer visibly as the suspect."})
            reply = self.chat(self.messages, temperature=self.temperature, max_tokens=self.max_tokens)
            self.messages.append({"role": "assistant", "content": reply})
            self.say("suspect: " + reply.replace(MARKER, "").strip())
            if confessed(reply):
                self.say("DEAD TO RIGHTS | the suspect confessed")
                return "confessed"
            trim_conversation(self.messages)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--model", default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--max-tokens", type=int, default=700)
    a = ap.parse_args()
    from ..client import DeliveranceClient

    client = DeliveranceClient(a.url)

    def chat(messages, **fields):
        if a.model:
            fields["model"] = a.model
        j = client.chat(messages, **fields)
        if "error" in j:
            raise RuntimeError(j["error"].get("message", "server error"))
        return j["choices"][0]["message"].get("content") or ""

    def ask():
        print("\ninterrogate> ", end="", flush=True)
        line = sys.stdin.readline()
        return line if line else None

    Game(chat, ask, print, a.seed, a.temperature, a.max_tokens).play()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
