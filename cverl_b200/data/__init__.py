"""Datasets: prompt/answer JSONL files read by the native host library."""
from .jsonl import PromptAnswerExample, load_prompt_answer_jsonl, download_hf_dataset  # noqa: F401
