// Constants that the kernels, the native host library and (through the host library) the Python
// layer must agree on. MythEclipse/llm keeps its plan constants in code as well
// (apps/engine/src/session.rs:10-21, tactics.rs:189-198, cuda/mod.rs:71-73); here they have one home.
#pragma once

#define LLMB_PAGE 64            // positions per cache page: the unit of the page pools and page tables
#define LLMB_GLU_BLOCK 16       // gate and up rows alternate in blocks of this many rows where the
                                // gated activation runs in the product's epilogue
#define LLMB_MAX_HEAD_DIM 256   // largest head size any attention kernel takes
