"""Micro-services around the engines: data, inference, training, agent and weight-update
services. Each follows the same shape as in the reference (``areal/infra/data_service``,
``areal/experimental/{inference,training,agent}_service``, ``areal/experimental/weight_update``):
a *gateway* (authentication, public routes), a *router* (worker registry + placement strategy)
and *workers* that do the work; ``base`` holds what they share."""
