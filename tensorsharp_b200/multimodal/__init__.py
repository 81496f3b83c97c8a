"""Vision and audio front ends: image processors, ViT-style encoders, the Gemma 4 audio conformer,
and the injector that splices their embeddings into a prompt.

Parity: TensorSharp.Models/Models/*/…VisionEncoder.cs, …ImageProcessor.cs,
Gemma4Audio{Encoder,Preprocessor}.cs, ModelMultimodalInjector.cs, MediaHelper.cs.  The encoders
run once per attachment (their output is cached by path + size + mtime), so they are written with
PyTorch tensor ops on the compute device; the language model's hot path never touches them.
"""
