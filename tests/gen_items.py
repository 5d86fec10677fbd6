"""Picklable generation items for the generation-controller tests (worker processes import this module)."""
import asyncio

from steptronoss_b200.generation.base_generatable import GenableItem, TrainableItem


class Square(GenableItem):
    def __init__(self, x, delay=0.0):
        super().__init__({"x": x})
        self.x, self.delay = x, delay

    async def generate(self):
        await asyncio.sleep(self.delay)
        if self.x < 0:
            raise ValueError("negative")
        return self.x * self.x


class Rollout(TrainableItem):
    def __init__(self, x):
        super().__init__()
        self.x = x

    async def generate(self):
        return self.x

    async def generate_for_train(self):
        return [self.x, self.x + 1]
