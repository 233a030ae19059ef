// Stand-in for a Faiss header (Faiss is not installed here); see faiss/Index.h.
#pragma once
#include <faiss/Index.h>
