"""B200-native inference engine for the Llama dense decoder (one GPU).

    from cisr_b200 import Model, Engine, Request
    model = Model.from_pretrained("path/to/model", dtype="bfloat16")    # or Model.from_config("smollm2-135m", seed=0)
    engine = Engine.for_model(model, pages=1024, page_size=16)
    engine.submit(Request("a", prompt=[1, 2, 3], max_new_tokens=16))
    for request in engine.run():
        print(request.key, request.generated)
"""
from .config import LlamaConfig, register_architecture
from .engine import Engine, Model, Request, StepEntry, Stepper

__all__ = ["Engine", "LlamaConfig", "Model", "Request", "StepEntry", "Stepper", "register_architecture"]
