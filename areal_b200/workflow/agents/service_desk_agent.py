"""Customer-service desk tasks in the style of tau-bench: the policy is the agent at an airline's service desk. A
simulated customer with a goal talks to it; the agent looks things up and changes a small reservation database
through tools, and has to follow a written policy that the tools do NOT enforce (a cancellation the policy forbids
goes through, and costs the reward). The episode is rewarded by the final state of the database: it must equal the
state that the task's reference actions produce from the same start, and the agent must have told the customer
what the task lists under ``outputs``.

A task is ``{"user_id", "opening", "facts": {keyword: reply}, "db": {...}, "expected_actions": [{"name",
"arguments"}], "outputs": [str]}`` (``make_desk_tasks`` generates them; a JSONL file of such records loads through
``dataset/agent_tasks.py``). The customer is :class:`ScriptedUser` (answers the agent's questions from ``facts`` by
keyword; deterministic, needs no second model) or :class:`LLMUser` (another chat endpoint playing the customer from
the scenario text, as tau-bench does).

Reference behaviour: examples/tau2/{agent.py,utils.py,train.py} (agent + user simulator + domain tools from the
tau2 package, reward from the domain's evaluator; every agent completion of the episode is a training sample).
That package is not available here, so the domain below is this repository's own.
"""

from __future__ import annotations

import copy
import json
import random
from typing import Any

from .math_agent import _client, _get, _message_dict
from .search_agent import _tool

STOP = "###STOP###"

DESK_POLICY = """You are a customer service agent of an airline. Help the customer with their reservation.
Rules you must follow:
1. Identify the customer by user id and look the reservation up before changing anything.
2. A reservation may be cancelled only if it was booked within the last 24 hours, or it is in business class, or it
   has travel insurance. Otherwise refuse the cancellation and explain why.
3. Basic economy reservations cannot be moved to another flight. Other reservations can be moved to a flight with the
   same origin and destination that still has seats.
4. Checked bags can be added, never removed.
5. Make one tool call at a time. Before a call that changes the database, state what you will do and obtain the
   customer's explicit confirmation.
6. If a request is outside these rules, transfer to a human agent.
When the customer's requests are handled, say goodbye."""

DESK_TOOLS = [
    _tool("get_user_details", "Profile of a customer and the ids of their reservations.", {"user_id": "string"}),
    _tool("get_reservation_details", "Flight, cabin, insurance, bags and status of a reservation.",
          {"reservation_id": "string"}),
    _tool("search_flights", "Flights between two airports on a date (YYYY-MM-DD) with price and free seats.",
          {"origin": "string", "destination": "string", "date": "string"}),
    _tool("cancel_reservation", "Cancel a reservation.", {"reservation_id": "string"}),
    _tool("change_flight", "Move a reservation to another flight.",
          {"reservation_id": "string", "flight_number": "string"}),
    _tool("update_baggage", "Set the total number of checked bags of a reservation.",
          {"reservation_id": "string", "total_bags": "integer"}),
    _tool("transfer_to_human_agent", "Hand the conversation to a human agent with a summary.", {"summary": "string"}),
]

WRITE_TOOLS = {"cancel_reservation", "change_flight", "update_baggage"}


class DeskDB:
    """The domain's state and tools. Tools keep the data consistent (ids exist, seats are counted) and nothing more:
    following the policy is the agent's job."""

    def __init__(self, data: dict[str, Any]):
        self.data = copy.deepcopy(data)

    def call(self, name: str, arguments: str | dict) -> str:
        try:
            args = json.loads(arguments) if isinstance(arguments, str) else dict(arguments or {})
            fn = getattr(self, "_" + name, None)
            if fn is None or name.startswith("_"):
                return f"error: unknown tool {name!r}"
            return json.dumps(fn(**args), sort_keys=True)
        except Exception as e:  # noqa: BLE001 - reported back to the model
            return f"error: {type(e).__name__}: {e}"

    def _res(self, reservation_id: str) -> dict:
        r = self.data["reservations"].get(str(reservation_id))
        if r is None:
            raise KeyError(f"no reservation {reservation_id}")
        return r

    def _get_user_details(self, user_id: str):
        u = self.data["users"].get(str(user_id))
        if u is None:
            raise KeyError(f"no user {user_id}")
        return dict(u, reservations=sorted(k for k, r in self.data["reservations"].items() if r["user_id"] == user_id))

    def _get_reservation_details(self, reservation_id: str):
        r = self._res(reservation_id)
        return dict(r, flight=dict(self.data["flights"][r["flight_number"]], flight_number=r["flight_number"]))

    def _search_flights(self, origin: str, destination: str, date: str):
        return [dict(f, flight_number=no) for no, f in sorted(self.data["flights"].items())
                if (f["origin"], f["destination"], f["date"]) == (origin, destination, date)]

    def _cancel_reservation(self, reservation_id: str):
        r = self._res(reservation_id)
        if r["status"] == "cancelled":
            raise ValueError("already cancelled")
        r["status"] = "cancelled"
        self.data["flights"][r["flight_number"]]["seats"] += 1
        return {"status": "cancelled"}

    def _change_flight(self, reservation_id: str, flight_number: str):
        r = self._res(reservation_id)
        new, old = self.data["flights"].get(flight_number), self.data["flights"][r["flight_number"]]
        if new is None:
            raise KeyError(f"no flight {flight_number}")
        if r["status"] != "active" or new["seats"] <= 0:
            raise ValueError("reservation is not active or the flight is full")
        if (new["origin"], new["destination"]) != (old["origin"], old["destination"]):
            raise ValueError("origin and destination must stay the same")
        old["seats"] += 1
        new["seats"] -= 1
        r["flight_number"] = flight_number
        return {"flight_number": flight_number, "price_difference": new["price"] - old["price"]}

    def _update_baggage(self, reservation_id: str, total_bags: int):
        r = self._res(reservation_id)
        r["bags"] = int(total_bags)
        return {"bags": r["bags"]}

    def _transfer_to_human_agent(self, summary: str = ""):
        self.data.setdefault("transfers", []).append(str(summary)[:200] and "transferred")
        return {"transferred": True}


def expected_state(task: dict) -> dict:
    db = DeskDB(task["db"])
    for a in task.get("expected_actions") or []:
        out = db.call(a["name"], a.get("arguments") or {})
        assert not out.startswith("error:"), (a, out)
    return db.data


def desk_reward(task: dict, final_db: dict, agent_messages: list[str]) -> float:
    """1.0 iff the database ended in the reference state and every required piece of information was said."""
    if final_db != expected_state(task):
        return 0.0
    said = " ".join(agent_messages).lower()
    return float(all(str(o).lower() in said for o in task.get("outputs") or []))


class ScriptedUser:
    """Answers from the task's ``facts``: the first keyword that occurs in the agent's message selects the reply
    (each fact is given once); a request for confirmation is confirmed; when nothing is left to say, or the agent
    says goodbye, the customer ends the conversation."""

    def __init__(self, task: dict):
        self.task, self.given = task, set()

    def opening(self) -> str:
        return self.task["opening"]

    async def respond(self, agent_text: str) -> str:
        low = agent_text.lower()
        if any(w in low for w in ("goodbye", "have a nice", "anything else")):
            return STOP
        for key, reply in (self.task.get("facts") or {}).items():
            if key.lower() in low and key not in self.given:
                self.given.add(key)
                return reply
        if any(w in low for w in ("confirm", "shall i", "do you want me", "proceed", "would you like me")):
            return "Yes, please go ahead."
        return STOP


class LLMUser:
    """Another model plays the customer from the scenario text; it ends the conversation with ``###STOP###``."""

    def __init__(self, task: dict, client, model: str = "default", **sampling):
        self.task, self.client, self.model, self.sampling = task, client, model, sampling
        self.messages = [{"role": "system", "content": (
            "You are a customer contacting an airline's service desk. Scenario: " + task.get("scenario", task["opening"])
            + " Facts you know: " + json.dumps(task.get("facts") or {}) + " Answer the agent's questions briefly, "
            "reveal facts only when asked, and write " + STOP + " when your request has been handled or refused.")}]

    def opening(self) -> str:
        return self.task["opening"]

    async def respond(self, agent_text: str) -> str:
        self.messages.append({"role": "user", "content": agent_text})
        comp = await self.client.chat.completions.create(messages=self.messages, model=self.model, **self.sampling)
        text = _get(comp.choices[0].message, "content") or STOP
        self.messages.append({"role": "assistant", "content": text})
        return text


class ServiceDeskAgent:
    def __init__(self, max_turns: int = 20, user: str = "scripted", user_client=None, **sampling):
        self.max_turns, self.user_kind, self.user_client = max_turns, user, user_client
        self.sampling = {k: v for k, v in sampling.items() if k != "max_tokens"}

    def _user(self, task: dict):
        if self.user_kind == "llm":
            if self.user_client is None:
                raise ValueError("user='llm' needs `user_client` (an OpenAI-compatible async client)")
            return LLMUser(task, self.user_client)
        return ScriptedUser(task)

    async def run(self, data: dict, **extra) -> float:
        client = _client(extra)
        db, user = DeskDB(data["db"]), self._user(data)
        messages = [{"role": "system", "content": DESK_POLICY}, {"role": "user", "content": user.opening()}]
        said: list[str] = []
        for _ in range(self.max_turns):
            comp = await client.chat.completions.create(messages=messages, model="default", tools=DESK_TOOLS,
                                                        **self.sampling)
            message = comp.choices[0].message
            messages.append(_message_dict(message))
            calls = _get(message, "tool_calls") or []
            if calls:
                for c in calls:
                    fn = _get(c, "function")
                    messages.append({"role": "tool", "tool_call_id": _get(c, "id"),
                                     "content": db.call(_get(fn, "name"), _get(fn, "arguments"))})
                continue
            text = _get(message, "content") or ""
            said.append(text)
            reply = await user.respond(text)
            if STOP in reply:
                break
            messages.append({"role": "user", "content": reply})
        return desk_reward(data, db.data, said)


# --------------------------------------------------------------------------- task generation

_AIRPORTS = ["SFO", "JFK", "SEA", "ORD", "ATL", "DFW", "BOS", "LAX"]


def make_desk_tasks(n: int, seed: int = 0) -> list[dict]:
    """Scenarios of four kinds: a cancellation the policy allows, one it forbids (reference: no action), a move to
    the cheapest flight of the day, added bags."""
    rng = random.Random(seed)
    tasks = []
    for i in range(n):
        kind = ("cancel_ok", "cancel_refuse", "change", "bags")[i % 4]
        uid, rid = f"user_{rng.randrange(1000, 9999)}", f"R{rng.randrange(10000, 99999)}"
        a, b = rng.sample(_AIRPORTS, 2)
        date = f"2025-{rng.randrange(1, 13):02d}-{rng.randrange(1, 28):02d}"
        flights = {f"AB{100 + j}": {"origin": a, "destination": b, "date": date, "price": rng.randrange(90, 600),
                                    "seats": rng.randrange(1, 9)} for j in range(4)}
        mine = rng.choice(sorted(flights))
        cabin = {"cancel_ok": rng.choice(["business", "economy"]), "cancel_refuse": "economy", "bags": "economy",
                 "change": "economy"}[kind]
        res = {"user_id": uid, "flight_number": mine, "cabin": cabin, "status": "active", "bags": rng.randrange(0, 2),
               "insurance": kind == "cancel_ok" and cabin == "economy",
               "booked_hours_ago": rng.randrange(30, 400)}
        db = {"users": {uid: {"name": f"Customer {i}", "membership": rng.choice(["regular", "silver", "gold"])}},
              "reservations": {rid: res}, "flights": flights}
        facts = {"user id": f"My user id is {uid}.", "reservation": f"The reservation is {rid}."}
        if kind in ("cancel_ok", "cancel_refuse"):
            opening = "Hi, I need to cancel my flight."
            actions = [{"name": "cancel_reservation", "arguments": {"reservation_id": rid}}] if kind == "cancel_ok" else []
            outputs = [] if kind == "cancel_ok" else []
        elif kind == "change":
            others = {k: f for k, f in flights.items() if k != mine}
            best = min(sorted(others), key=lambda k: others[k]["price"])
            opening = "Hello, I'd like to move my reservation to the cheapest other flight on the same day."
            facts["which flight"] = f"Whichever other flight is cheapest that day, so {best} if I read the site right."
            actions = [{"name": "change_flight", "arguments": {"reservation_id": rid, "flight_number": best}}]
            outputs = [best]
        else:
            total = res["bags"] + rng.randrange(1, 3)
            opening = "Hi, I want to bring more checked bags."
            facts["how many"] = f"I need {total} checked bags in total."
            actions = [{"name": "update_baggage", "arguments": {"reservation_id": rid, "total_bags": total}}]
            outputs = [str(total)]
        tasks.append({"task_id": f"desk-{seed}-{i}", "kind": kind, "user_id": uid, "opening": opening, "facts": facts,
                      "scenario": f"{opening} (kind: {kind})", "db": db, "expected_actions": actions,
                      "outputs": outputs, "messages": [{"role": "user", "content": opening}]})
    return tasks
