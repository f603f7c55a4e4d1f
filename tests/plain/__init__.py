"""Plain, slow restatement of the Qwen2.5 dense decoder used as the test oracle.

Nothing here imports the engine package: it has its own config reading, its own
safetensors reader and one function for each part of the model.
"""
