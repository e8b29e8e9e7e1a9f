"""Typed configurations and the architecture-neutral model plan."""

from .model_plan import LayerSpec, ModelPlan, PartSpec, RunEntry, schedule_from_lists, sequential_schedule

__all__ = ["LayerSpec", "ModelPlan", "PartSpec", "RunEntry", "schedule_from_lists", "sequential_schedule"]
