// <faiss/ascend/AscendClonerOptions.h>: install path the reference's clients include.  The declarations of all
// faiss::ascend classes of the B200 search path live in one header.
#pragma once
#include "../../b200/ascend_api.h"
