#pragma once
#include "COO.hpp"
#include "CSR.hpp"
#include "Dense.hpp"
#include "triplet.h"
